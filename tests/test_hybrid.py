"""Hybrid (gated-DeltaNet) graph on the CPU oracle path: chunked prefill consistency, streaming conv state,
MTP self-speculative decoding being lossless with full / partial / no acceptance (the reference's checks:
tools/ie_validate_chunking.cpp, tools/ie_qwen35_spec.cpp, tools/ie_spec_engine_ab.cpp)."""
import torch

from machx_inference_engine_b200 import ops
from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.models import build_model
from machx_inference_engine_b200.runtime.engine import EngineOptions, LLMEngine, SamplingParams


def _model(name="tiny-qwen3next"):
    return build_model(preset(name), "cpu", quant="q8_0", max_ctx=512)


def test_conv1d_streaming_equals_one_shot():
    torch.manual_seed(0)
    T, C, Kc = 23, 64, 4
    x = torch.randn(T, C).to(torch.bfloat16)
    w = torch.randn(C, Kc)
    slots = torch.tensor([1], dtype=torch.int32)
    st = torch.zeros(3, Kc - 1, C, dtype=torch.bfloat16)
    full = ops.conv1d_silu(x, w, st, slots, torch.tensor([0, T], dtype=torch.int32), T)
    st2 = torch.zeros(3, Kc - 1, C, dtype=torch.bfloat16)
    parts, t = [], 0
    for n in (5, 1, 1, 9, 2, 5):
        parts.append(ops.conv1d_silu(x[t:t + n], w, st2, slots, torch.tensor([0, n], dtype=torch.int32), n))
        t += n
    assert torch.equal(full, torch.cat(parts))
    assert torch.equal(st, st2) and torch.equal(st[1], x[-(Kc - 1):])
    # direct definition: tap j multiplies input t-(Kc-1)+j
    xf = torch.cat([torch.zeros(Kc - 1, C), x.float()])
    want = torch.stack([(xf[i:i + Kc].T * w).sum(-1) for i in range(T)])
    assert torch.allclose(full.float(), torch.nn.functional.silu(want), atol=2e-2, rtol=2e-2)


def test_deltanet_scan_chunked_state_and_checkpoints():
    torch.manual_seed(1)
    n_k, n_v, T, D = 2, 4, 19, 128
    qkv = torch.randn(T, (2 * n_k + n_v) * D).to(torch.bfloat16)
    ab = torch.randn(T, 2 * n_v).to(torch.bfloat16)
    a_idx = torch.arange(n_v, dtype=torch.int32)
    b_idx = a_idx + n_v
    k_of_v = torch.tensor([0, 0, 1, 1], dtype=torch.int32)
    ssm_a = -torch.rand(n_v) - 0.1
    dtb = torch.randn(n_v) * 0.1
    slots = torch.tensor([0], dtype=torch.int32)
    S1 = torch.zeros(1, n_v, D, D)
    ck = torch.zeros(T, n_v, D, D)
    full = ops.deltanet_scan(qkv, n_k, ab, a_idx, b_idx, k_of_v, ssm_a, dtb, S1, slots, torch.tensor([0, T], dtype=torch.int32), n_v, ckpt=ck)
    S2 = torch.zeros(1, n_v, D, D)
    outs, t = [], 0
    for n in (7, 1, 11):
        outs.append(ops.deltanet_scan(qkv[t:t + n], n_k, ab[t:t + n], a_idx, b_idx, k_of_v, ssm_a, dtb, S2, slots,
                                      torch.tensor([0, n], dtype=torch.int32), n_v))
        t += n
        assert torch.allclose(S2[0], ck[t - 1], atol=1e-5)
    assert torch.allclose(full, torch.cat(outs), atol=1e-5)
    assert torch.allclose(S1, S2, atol=1e-5)


def test_chunked_prefill_matches_whole_prompt():
    m = _model()
    prompt = [(i * 7 + 3) % m.cfg.vocab for i in range(37)]
    grabbed = {}
    for chunk in (512, 16):
        eng = LLMEngine(m, EngineOptions(max_ctx=512, max_batch_tokens=chunk, max_seqs=2))
        seq = eng.add_request(prompt, SamplingParams(max_tokens=2, ignore_eos=True))
        orig, got = m.forward, []
        m.forward = lambda *a, **k: (got.append(orig(*a, **k)), got[-1])[1]
        try:
            while seq.n_generated < 1:
                eng.step()
        finally:
            m.forward = orig
        grabbed[chunk] = got[-1][-1]
    cos = torch.nn.functional.cosine_similarity(grabbed[512], grabbed[16], dim=0)
    assert cos > 0.9995


def test_dense_hybrid_tiled_heads_chunked_and_spec():
    """Qwen3.6-27B-style graph: dense FFN, (1 + w) norms, tiled k->v head repeat, separate alpha / beta projections."""
    m = _model("tiny-qwen35")
    assert m.one_plus_w and m.mtp is not None
    prompt = [(i * 13 + 5) % m.cfg.vocab for i in range(41)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    whole = LLMEngine(m, EngineOptions(max_ctx=512, max_seqs=2)).generate([prompt], sp)[0]
    spec = LLMEngine(m, EngineOptions(max_ctx=512, max_seqs=2, spec_k=2)).generate([prompt], sp)[0]
    assert whole == spec
    chunked = LLMEngine(m, EngineOptions(max_ctx=512, max_seqs=2, max_batch_tokens=16)).generate([prompt], sp)[0]
    assert chunked[:2] == whole[:2]


def test_two_sequences_keep_separate_state():
    m = _model()
    p1 = [(i * 5 + 1) % m.cfg.vocab for i in range(21)]
    p2 = [(i * 11 + 2) % m.cfg.vocab for i in range(33)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    solo = [LLMEngine(m, EngineOptions(max_ctx=512, max_seqs=2)).generate([p], sp)[0] for p in (p1, p2)]
    both = LLMEngine(m, EngineOptions(max_ctx=512, max_seqs=2)).generate([p1, p2], sp)
    assert both[0][:3] == solo[0][:3] and both[1][:3] == solo[1][:3]


def test_spec_decode_is_lossless_with_any_acceptance():
    m = _model()
    V = m.cfg.vocab
    prompt = [(i * 7 + 3) % V for i in range(37)]
    sp = SamplingParams(max_tokens=20, ignore_eos=True)
    truth = LLMEngine(m, EngineOptions(max_ctx=512, max_seqs=2)).generate([prompt], sp)[0]
    # the model's own (random-init) head: drafts are wrong, every round rolls back to the first position
    eng = LLMEngine(m, EngineOptions(max_ctx=512, max_seqs=2, spec_k=3))
    assert eng.generate([prompt], sp)[0] == truth
    assert eng.stats["spec_rounds"] > 0
    # oracle drafts with 0..3 correct tokens in rotation: commits at every checkpoint row
    eng = LLMEngine(m, EngineOptions(max_ctx=512, max_seqs=2, spec_k=3))
    seq = eng.add_request(prompt, sp)
    rnd = [0]
    real = m.mtp.draft

    def fake(h, tok, k, ctx=None):
        g = len(seq.tokens) - len(prompt)
        d = (list(truth[g:g + k]) + [0] * k)[:k]
        rnd[0] += 1
        if rnd[0] % 4 < k:
            d[rnd[0] % 4] = (d[rnd[0] % 4] + 1) % V
        return d
    m.mtp.draft = fake
    try:
        while not seq.finished:
            eng.step()
    finally:
        m.mtp.draft = real
    assert seq.tokens[len(prompt):] == truth
    assert eng.stats["spec_accepted"] > 0 and eng.stats["spec_rounds"] < len(truth)


def test_prefix_cache_restores_recurrent_state():
    """A second request sharing a 256-token prefix resumes from the KV blocks AND the DeltaNet state saved at that boundary
    (the reference keeps a state snapshot per prefix-trie endpoint); its continuation must equal a cold run."""
    m = _model()
    V = m.cfg.vocab
    shared = [(i * 13 + 1) % V for i in range(300)]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    cold = LLMEngine(m, EngineOptions(max_ctx=1024, max_seqs=2, max_batch_tokens=128, enable_prefix_cache=False)).generate([shared + [5, 6, 7]], sp)[0]
    eng = LLMEngine(m, EngineOptions(max_ctx=1024, max_seqs=2, max_batch_tokens=128))
    first = eng.generate([shared + [9, 9]], sp)[0]
    assert len(eng.state_cache) == 2                       # snapshots after 128 and 256 prompt tokens
    pre = eng.stats["prefill_tokens"]
    seq = eng.add_request(shared + [5, 6, 7], sp)
    while not seq.finished:
        eng.step()
    assert seq.n_cached_prefix == 256 and eng.stats["prefill_tokens"] - pre == len(shared) + 3 - 256
    assert seq.tokens[len(seq.prompt):] == cold
    # a prefix whose blocks are cached but whose snapshot was evicted falls back to the longest boundary that has one
    eng.state_cache.popitem(last=True)
    seq = eng.add_request(shared + [5, 6, 7], sp)
    while not seq.finished:
        eng.step()
    assert seq.n_cached_prefix == 128 and seq.tokens[len(seq.prompt):] == cold


def test_deferred_admission_keeps_its_state_snapshot():
    """A request matches a cached prefix, cannot be admitted for a while (the block pool is held by another request), and in the
    meantime the recurrent-state snapshot of that prefix is pushed out of the LRU cache.  It must still resume from the state that
    belongs to its prefix (the sequence holds the snapshot from match to restore) and produce what a cold run produces."""
    m = _model()
    V = m.cfg.vocab
    shared = [(i * 13 + 1) % V for i in range(300)]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    cold = LLMEngine(m, EngineOptions(max_ctx=1024, max_seqs=2, max_batch_tokens=128, enable_prefix_cache=False)).generate([shared + [5, 6, 7]], sp)[0]
    # six usable blocks: two stay cached for the shared prefix, the blocker takes the other four
    eng = LLMEngine(m, EngineOptions(max_ctx=1024, max_seqs=2, max_batch_tokens=256, num_blocks=7))
    eng.generate([shared + [9, 9]], sp)
    assert len(eng.state_cache) == 1                        # one 256-token chunk: one snapshot, at the 256-token boundary
    blocker = eng.add_request([(i * 7 + 3) % V for i in range(484)], SamplingParams(max_tokens=4, ignore_eos=True))
    eng.step()                                              # first 256 tokens of the blocker
    late = eng.add_request(shared + [5, 6, 7], sp)
    eng.step()                                              # the blocker's rest leaves 28 tokens of budget: `late` matches, finds no block
    assert late in eng.sched.waiting and late.restore_hash is not None and late.n_cached_prefix == 256
    eng.state_cache.clear()                                 # what other traffic does to a 12-entry LRU in the meantime
    while not late.finished:
        eng.step()
    assert blocker.finished and late.tokens[len(late.prompt):] == cold
