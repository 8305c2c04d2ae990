"""Gated-DeltaNet kernels (conv1d+SiLU, delta-rule scan, per-head gated RMSNorm) and the hybrid graph against the
PyTorch fp32 oracle; mirrors tests/unit/deltanet_test.cpp, conv1d_test.cpp and the chunking validator of the reference."""
import pytest
import torch

from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.models import build_model
from machx_inference_engine_b200.ops import ref
from machx_inference_engine_b200.runtime.engine import EngineOptions, LLMEngine, SamplingParams

pytestmark = pytest.mark.gpu


def K():
    from machx_inference_engine_b200.ops import cuda
    return cuda


D = torch.device("cuda:0")


def rel_err(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).norm() / (b.norm() + 1e-12))


@pytest.mark.parametrize("lens,Kc", [([37], 4), ([1, 1, 1], 4), ([5, 1, 130, 2], 4), ([3, 2], 3), ([70, 201], 4), ([100, 1, 30], 3)])
def test_conv1d_silu(lens, Kc):
    torch.manual_seed(0)
    C, pad = 384, 40
    T, B = sum(lens), len(lens)
    xw = torch.randn(T, C + pad).to(torch.bfloat16)
    w = torch.randn(C, Kc)
    st = torch.randn(B + 2, Kc - 1, C).to(torch.bfloat16)
    slots = torch.tensor([i + 1 for i in range(B)], dtype=torch.int32)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    ck_ref = torch.zeros(T, Kc - 1, C, dtype=torch.bfloat16)
    st_ref = st.clone()
    want = ref.conv1d_silu(xw[:, :C], w, st_ref, slots, cu, max(lens), ckpt=ck_ref)
    st_g, ck_g = st.to(D), torch.zeros(T, Kc - 1, C, dtype=torch.bfloat16, device=D)
    got = K().conv1d_silu(xw.to(D)[:, :C], w.to(D), st_g, slots.to(D), cu.to(D), max(lens), ckpt=ck_g)
    assert rel_err(got, want) < 1e-2
    assert torch.equal(st_g.cpu(), st_ref)
    assert torch.equal(ck_g.cpu(), ck_ref)


@pytest.mark.parametrize("lens", [[1], [1, 1, 1, 1], [19], [16, 33, 1], [300]])
def test_deltanet_scan(lens):
    torch.manual_seed(1)
    n_k, n_v, Dh = 2, 4, 128
    T, B = sum(lens), len(lens)
    qkv = torch.randn(T, (2 * n_k + n_v) * Dh).to(torch.bfloat16)
    ab = torch.randn(T, 2 * n_v + 8).to(torch.bfloat16)
    b_idx = torch.tensor([0, 1, 4, 5], dtype=torch.int32)          # fused per-k-head [beta, beta, alpha, alpha] groups
    a_idx = b_idx + 2
    k_of_v = torch.tensor([0, 0, 1, 1], dtype=torch.int32)
    ssm_a = -torch.rand(n_v) - 0.05
    dtb = torch.randn(n_v) * 0.2
    slots = torch.tensor(list(range(B, 0, -1)), dtype=torch.int32)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    S0 = torch.randn(B + 1, n_v, Dh, Dh) * 0.05
    S_ref, ck_ref = S0.clone(), torch.zeros(T, n_v, Dh, Dh)
    want = ref.deltanet_scan(qkv, n_k, ab, a_idx, b_idx, k_of_v, ssm_a, dtb, S_ref, slots, cu, n_v, ckpt=ck_ref)
    S_g = S0.to(D)
    use_ck = T <= 64
    ck_g = torch.zeros(T, n_v, Dh, Dh, device=D) if use_ck else None
    got = K().deltanet_scan(qkv.to(D), n_k, ab.to(D), a_idx.to(D), b_idx.to(D), k_of_v.to(D), ssm_a.to(D), dtb.to(D), S_g, slots.to(D), cu.to(D),
                            n_v, ckpt=ck_g, chunked=False)
    assert rel_err(got, want) < 2e-3
    assert rel_err(S_g, S_ref) < 2e-3
    if use_ck:
        assert rel_err(ck_g, ck_ref) < 2e-3


@pytest.mark.parametrize("lens", [[64], [300], [130, 1, 70], [640, 200]])
def test_deltanet_scan_chunked_tensor_core(lens):
    """The chunked (WY) scan on the tensor cores against the sequential fp32 recurrence: outputs and final state, ragged chunk
    boundaries, several sequences, a non-zero initial state, and a second call that carries the state on.  Its operands are bf16
    (the state as a hi + lo pair), so the tolerance is the bf16 one."""
    torch.manual_seed(7)
    n_k, n_v, Dh = 2, 4, 128
    T, B = sum(lens), len(lens)
    qkv = torch.randn(T, (2 * n_k + n_v) * Dh).to(torch.bfloat16)
    ab = torch.randn(T, 2 * n_v + 8).to(torch.bfloat16)
    b_idx = torch.tensor([0, 1, 4, 5], dtype=torch.int32)
    a_idx = b_idx + 2
    k_of_v = torch.tensor([0, 0, 1, 1], dtype=torch.int32)
    ssm_a = -torch.rand(n_v) - 0.05
    dtb = torch.randn(n_v) * 0.2
    slots = torch.tensor(list(range(B, 0, -1)), dtype=torch.int32)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    S0 = torch.randn(B + 1, n_v, Dh, Dh) * 0.05
    S_ref = S0.clone()
    want = ref.deltanet_scan(qkv, n_k, ab, a_idx, b_idx, k_of_v, ssm_a, dtb, S_ref, slots, cu, n_v)
    g = lambda t: t.to(D)
    S_g = S0.to(D)
    got = K().deltanet_scan(g(qkv), n_k, g(ab), g(a_idx), g(b_idx), g(k_of_v), g(ssm_a), g(dtb), S_g, g(slots), g(cu), n_v, chunked=True)
    K().check_status()
    assert rel_err(got, want) < 1e-2, rel_err(got, want)
    assert rel_err(S_g, S_ref) < 5e-3, rel_err(S_g, S_ref)
    assert torch.equal(S_g[0].cpu(), S0[0])                                  # a slot no sequence uses is untouched
    # the oracle's own chunked restatement agrees with the recurrence to fp32 rounding
    S_c = S0.clone()
    alt = ref.deltanet_scan_chunked(qkv, n_k, ab, a_idx, b_idx, k_of_v, ssm_a, dtb, S_c, slots, cu, n_v)
    assert rel_err(alt, want) < 1e-5 and rel_err(S_c, S_ref) < 1e-5
    # carry: the same tokens again, continuing from the state the first call left
    want2 = ref.deltanet_scan(qkv, n_k, ab, a_idx, b_idx, k_of_v, ssm_a, dtb, S_ref, slots, cu, n_v)
    got2 = K().deltanet_scan(g(qkv), n_k, g(ab), g(a_idx), g(b_idx), g(k_of_v), g(ssm_a), g(dtb), S_g, g(slots), g(cu), n_v, chunked=True)
    K().check_status()
    assert rel_err(got2, want2) < 1.5e-2 and rel_err(S_g, S_ref) < 1e-2


def test_gated_rmsnorm_heads_strided_z():
    torch.manual_seed(2)
    T, n_h, hd = 9, 4, 128
    x = torch.randn(T, n_h * hd)
    zw = torch.randn(T, 100 + n_h * hd + 12).to(torch.bfloat16)
    w = torch.rand(hd) + 0.5
    want = ref.gated_rmsnorm_heads(x, zw[:, 100:100 + n_h * hd], w, 1e-6, hd)
    got = K().gated_rmsnorm_heads(x.to(D), zw.to(D)[:, 100:100 + n_h * hd], w.to(D), 1e-6, hd)
    assert rel_err(got, want) < 1e-2


@pytest.mark.parametrize("spec_k", [0, 3])
def test_hybrid_model_matches_cpu_oracle(spec_k):
    """Greedy tokens of the engine on the GPU (plain and self-speculative) against the CPU oracle.  Random-init logits and router scores
    have near-ties, and one flipped token changes everything after it, so free-running continuations are compared only in their first
    token; the steps after it are compared one at a time from the oracle's own context: the GPU engine gets the prompt plus the oracle's
    first i tokens and must produce the oracle's next two (one from the prefill path, one from a decode step)."""
    cfg = preset("tiny-qwen3next")
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (37, 150)]
    cpu = LLMEngine(build_model(cfg, torch.device("cpu"), quant="q8_0", max_ctx=512, gen_device="cpu"), EngineOptions(max_ctx=512, max_batch_tokens=64, max_seqs=2))
    gpu = LLMEngine(build_model(cfg, torch.device("cuda:0"), quant="q8_0", max_ctx=512, gen_device="cpu"),
                    EngineOptions(max_ctx=512, max_batch_tokens=64, max_seqs=2, spec_k=spec_k))
    want = [cpu.generate([p], SamplingParams(max_tokens=10, ignore_eos=True))[0] for p in prompts]
    free = [gpu.generate([p], SamplingParams(max_tokens=10, ignore_eos=True))[0] for p in prompts]
    assert all(x[0] == y[0] and len(y) == 10 for x, y in zip(want, free)), (want, free)
    assert free == [gpu.generate([p], SamplingParams(max_tokens=10, ignore_eos=True))[0] for p in prompts]       # deterministic
    first = second = valid = total = 0
    for p, toks in zip(prompts, want):
        for i in range(0, len(toks) - 1):
            got = gpu.generate([p + toks[:i]], SamplingParams(max_tokens=2, ignore_eos=True))[0]
            total += 1
            first += int(got[0] == toks[i])
            if got[0] == toks[i]:
                valid += 1
                second += int(got[1] == toks[i + 1])
    assert first >= 0.75 * total and second >= 0.75 * valid, (first, second, valid, total)


@pytest.mark.parametrize("name", ["tiny-qwen35", "tiny-qwen3next"])
def test_hybrid_logits_cosine_chunked(name):
    """Teacher-forced logits over a prompt fed in three chunks (state carried between forwards) and six decode steps (the one-row
    GEMV / expert-GEMV path; its rows are also held to a bound of their own, since six rows would vanish in the mean over 206).
    The dense hybrid must agree row by row; with random-init routers the MoE hybrid can pick a different expert on a
    near-tie, which changes single rows, so it is held to the mean."""
    from machx_inference_engine_b200.models.transformer import KV_BLOCK, ForwardBatch
    cfg = preset(name)
    ids = torch.randint(0, cfg.vocab, (206,), generator=torch.Generator().manual_seed(1)).tolist()
    res = {}
    for dev in ("cpu", "cuda:0"):
        d = torch.device(dev)
        m = build_model(cfg, d, quant="q8_0", max_ctx=512, gen_device="cpu")
        kv, st = m.new_kv_cache(6), m.new_state(2)
        bt = torch.arange(1, 5, dtype=torch.int32, device=d).unsqueeze(0)
        outs, t0 = [], 0
        for n in (64, 72, 64, 1, 1, 1, 1, 1, 1):
            pos = torch.arange(t0, t0 + n, dtype=torch.int32, device=d)
            slot = bt[0][(pos // KV_BLOCK).long()].long() * KV_BLOCK + (pos % KV_BLOCK).long()
            fb = ForwardBatch(torch.tensor(ids[t0:t0 + n], dtype=torch.int32, device=d), pos, slot, bt,
                              torch.tensor([t0 + n], dtype=torch.int32, device=d), torch.tensor([0, n], dtype=torch.int32, device=d), n,
                              logit_rows=torch.arange(n, device=d), state_slots=torch.tensor([1], dtype=torch.int32, device=d),
                              state_slots_host=[1], start_host=[t0])
            outs.append(m.forward(fb, kv, st).float().cpu())
            t0 += n
        res[dev] = torch.cat(outs)
    a, b = res["cpu"], res["cuda:0"]
    cos = torch.nn.functional.cosine_similarity(a, b, dim=1)
    if name == "tiny-qwen35":
        assert float(cos.min()) > 0.995, cos
        assert (a.argmax(-1) == b.argmax(-1)).float().mean() > 0.9
    else:
        assert float(cos.mean()) > 0.98 and float(cos.median()) > 0.999, cos
        assert float(cos[-6:].median()) > 0.999 and float(cos[-6:].min()) > 0.9, cos[-6:]
