"""Gemma-4 graph against an independent plain-PyTorch restatement of the layer math (dense tensors read back from the file,
whole-sequence attention with explicit masks): config round trip, file path, chunked prefill, paged decode."""
import dataclasses
import math

import pytest
import torch

from machx_inference_engine_b200.formats.gguf import GGUFReader
from machx_inference_engine_b200.formats.model_config import preset, read_config
from machx_inference_engine_b200.formats.synth import write_synthetic_gguf
from machx_inference_engine_b200.models import load_model
from machx_inference_engine_b200.models.transformer import KV_BLOCK, ForwardBatch
from machx_inference_engine_b200.runtime.engine import EngineOptions, LLMEngine, SamplingParams


def _rms(x, w=None, eps=1e-6):
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def _rope(t, pos, n_rot, theta):
    half = n_rot // 2
    inv = theta ** (-torch.arange(0, n_rot, 2, dtype=torch.float64) / n_rot)
    ang = pos.to(torch.float64).unsqueeze(-1) * inv                       # [T, half]
    c, s = torch.cos(ang).float().unsqueeze(1), torch.sin(ang).float().unsqueeze(1)
    a, b = t[..., :half], t[..., half:n_rot]
    return torch.cat([a * c - b * s, a * s + b * c, t[..., n_rot:]], dim=-1)


def oracle_logits(path, ids):
    r = GGUFReader(path)
    c = read_config(r.kv, r.tensors.keys())
    W = lambda n: torch.from_numpy(r.tensor(n).to_float32().copy())
    T, H = len(ids), c.hidden
    pos = torch.arange(T)
    emb = W("token_embd.weight")
    x = emb[torch.tensor(ids)] * math.sqrt(H)
    for l in range(c.n_layers):
        p = f"blk.{l}."
        hd, n_kv, n_rot, theta = c.layer_geometry(l)
        h = _rms(x, W(p + "attn_norm.weight"))
        q = (h @ W(p + "attn_q.weight").T).reshape(T, c.n_heads, hd)
        kraw = (h @ W(p + "attn_k.weight").T).reshape(T, n_kv, hd)
        v = (h @ W(p + "attn_v.weight").T).reshape(T, n_kv, hd) if r.has_tensor(p + "attn_v.weight") else kraw
        q, k, v = _rms(q, W(p + "attn_q_norm.weight")), _rms(kraw, W(p + "attn_k_norm.weight")), _rms(v)
        q, k = _rope(q, pos, n_rot, theta), _rope(k, pos, n_rot, theta)
        rep = c.n_heads // n_kv
        s = torch.einsum("thd,shd->hts", q, k.repeat_interleave(rep, dim=1))          # scale 1
        ok = pos.unsqueeze(0) <= pos.unsqueeze(1)
        if c.layer_window(l):
            ok = ok & (pos.unsqueeze(0) > pos.unsqueeze(1) - c.layer_window(l))
        s = s.masked_fill(~ok.unsqueeze(0), float("-inf"))
        a = torch.einsum("hts,shd->thd", torch.softmax(s, -1), v.repeat_interleave(rep, dim=1)).reshape(T, c.n_heads * hd)
        a_out = x + _rms(a @ W(p + "attn_output.weight").T, W(p + "post_attention_norm.weight"))
        hn = _rms(a_out, W(p + "ffn_norm.weight"))
        gelu = lambda t: torch.nn.functional.gelu(t, approximate="tanh")
        y = (gelu(hn @ W(p + "ffn_gate.weight").T) * (hn @ W(p + "ffn_up.weight").T)) @ W(p + "ffn_down.weight").T
        if r.has_tensor(p + "ffn_gate_inp.weight"):
            y = _rms(y, W(p + "post_ffw_norm_1.weight"))
            e_in = _rms(a_out, W(p + "pre_ffw_norm_2.weight"))
            rin = _rms(a_out, W(p + "ffn_gate_inp.scale")) / math.sqrt(H)
            prob = torch.softmax(rin @ W(p + "ffn_gate_inp.weight").T, -1)
            top_p, top_i = prob.topk(c.n_experts_used, dim=-1)
            top_p = top_p / top_p.sum(-1, keepdim=True)
            gu, dn, ds = W(p + "ffn_gate_up_exps.weight"), W(p + "ffn_down_exps.weight"), W(p + "ffn_down_exps.scale").reshape(-1)
            F = c.expert_ffn
            m = torch.zeros(T, H)
            for t in range(T):
                for j in range(c.n_experts_used):
                    e = int(top_i[t, j])
                    gate_up = gu[e] @ e_in[t]
                    m[t] += float(top_p[t, j]) * float(ds[e]) * (dn[e] @ (gelu(gate_up[:F]) * gate_up[F:]))
            y = y + _rms(m, W(p + "post_ffw_norm_2.weight"))
        x = (a_out + _rms(y, W(p + "post_ffw_norm.weight"))) * float(W(p + "layer_output_scale.weight").reshape(-1)[0])
    logits = _rms(x, W("output_norm.weight")) @ emb.T
    return torch.tanh(logits / c.final_logit_softcap) * c.final_logit_softcap


def _forward_all(model, ids, chunk):
    """Logits of every position through the paged graph, in prefill chunks of `chunk` tokens."""
    nb = (len(ids) + KV_BLOCK - 1) // KV_BLOCK
    kv = model.new_kv_cache(nb + 1)
    bt = torch.arange(1, nb + 1, dtype=torch.int32).reshape(1, nb)
    out = []
    for lo in range(0, len(ids), chunk):
        hi = min(len(ids), lo + chunk)
        pos = torch.arange(lo, hi, dtype=torch.int32)
        slot = torch.tensor([int(bt[0, p // KV_BLOCK]) * KV_BLOCK + p % KV_BLOCK for p in range(lo, hi)], dtype=torch.int64)
        fb = ForwardBatch(torch.tensor(ids[lo:hi], dtype=torch.int32), pos, slot, bt, torch.tensor([hi], dtype=torch.int32),
                          torch.tensor([0, hi - lo], dtype=torch.int32), hi - lo, logit_rows=torch.arange(hi - lo))
        out.append(model.forward(fb, kv).float())
    return torch.cat(out)


@pytest.mark.parametrize("name", ["tiny-gemma4-dense", "tiny-gemma4"])
def test_graph_matches_plain_pytorch_oracle(tmp_path, name):
    cfg = preset(name)
    path = str(tmp_path / "g.gguf")
    write_synthetic_gguf(cfg, path, quant="bf16", seed=11)
    model, reader = load_model(path, torch.device("cpu"), max_ctx=1024)
    c = model.cfg
    assert c.arch == "gemma4" and c.layer_swa == cfg.layer_swa and c.layer_n_kv == cfg.layer_n_kv and c.head_dim_swa == cfg.head_dim_swa
    assert not reader.has_tensor("blk.2.attn_v.weight") and reader.has_tensor("blk.0.attn_v.weight")       # global layer: V = K projection
    assert model.kv_geometry == {0: (2, 64), 1: (2, 64), 2: (1, 128)}
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, c.vocab, (300,), generator=g).tolist()                # longer than the 128-token window and two pages
    want = oracle_logits(path, ids)
    for chunk in (300, 77):
        got = _forward_all(model, ids, chunk)
        cos = torch.nn.functional.cosine_similarity(got, want, dim=1)
        agree = float((got.argmax(-1) == want.argmax(-1)).float().mean())
        if cfg.is_moe:      # a near-tie in a router can still pick another expert for a token: assess the bulk, bound the tail
            assert float(cos.median()) > 0.999 and float((cos > 0.99).float().mean()) > 0.9 and agree > 0.85, (chunk, float(cos.median()), agree)
        else:
            assert float(cos.min()) > 0.998 and agree > 0.9, (chunk, float(cos.min()), agree)
    assert float(want.abs().max()) <= 30.0 and float(got.abs().max()) <= 30.0     # soft-cap


def test_engine_serves_gemma4_with_decode_and_int8_cache(tmp_path):
    cfg = preset("tiny-gemma4")
    path = str(tmp_path / "g.gguf")
    write_synthetic_gguf(cfg, path, quant="q8_0", seed=2)
    model, _ = load_model(path, torch.device("cpu"), max_ctx=1024)
    ids = list(range(10, 190))
    outs = {}
    for dt in ("bf16", "int8"):
        eng = LLMEngine(model, EngineOptions(max_ctx=1024, max_batch_tokens=64, max_seqs=2, kv_dtype=dt))
        assert eng.kv.k[2].shape[1:] == (1, KV_BLOCK, 128) and eng.kv.k[0].shape[1:] == (2, KV_BLOCK, 64)
        seq = eng.add_request(ids, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
        while not seq.finished:
            eng.step()
        outs[dt] = seq.tokens[len(ids):]
    # decode continues exactly where a longer prefill would: the 6 greedy tokens equal teacher-forced argmaxes
    full = ids + outs["bf16"]
    lg = _forward_all(model, full, len(full))
    assert [int(t) for t in lg[len(ids) - 1:len(full) - 1].argmax(-1)] == outs["bf16"]
    assert outs["int8"][0] == outs["bf16"][0]


def test_assistant_head_file_round_trip_and_lossless_spec_decode(tmp_path):
    """The gemma4-assistant draft head: its file format (metadata keys + tensors) loads, its queries read the target's cache (the head
    writes none), and greedy self-speculative decoding with it yields exactly the tokens of plain greedy decoding, whatever it drafts."""
    from machx_inference_engine_b200.formats.synth import write_synthetic_assistant_gguf
    from machx_inference_engine_b200.models.gemma4_assistant import load_assistant_head, read_assistant_config, synth_assistant_config
    from machx_inference_engine_b200.formats.gguf import GGUFReader
    cfg = preset("tiny-gemma4-dense")
    path, hpath = str(tmp_path / "g.gguf"), str(tmp_path / "head.gguf")
    write_synthetic_gguf(cfg, path, quant="q8_0", seed=3)
    acfg = synth_assistant_config(cfg, n_layers=3, hidden=128, ffn=256)
    assert acfg.is_swa == [True, True, False] and acfg.head_dim == [64, 64, 128] and acfg.n_kv_heads == [2, 2, 1]
    write_synthetic_assistant_gguf(acfg, hpath, quant="q8_0", seed=4)
    r = GGUFReader(hpath)
    back = read_assistant_config(r.kv, r.tensors)
    assert abs(back.rms_eps - acfg.rms_eps) < 1e-9 and dataclasses.replace(back, rms_eps=acfg.rms_eps) == acfg
    model, _ = load_model(path, torch.device("cpu"), max_ctx=512)
    ids = [(i * 11 + 5) % cfg.vocab for i in range(150)]
    sp = SamplingParams(max_tokens=14, temperature=0.0, ignore_eos=True)
    truth = LLMEngine(model, EngineOptions(max_ctx=512, max_batch_tokens=64, max_seqs=2)).generate([ids], sp)[0]
    head = load_assistant_head(model, hpath)
    assert model.mtp is head and [L["shared"] for L in head.layers] == [1, 1, 2]
    eng = LLMEngine(model, EngineOptions(max_ctx=512, max_batch_tokens=64, max_seqs=2, spec_k=3))
    assert eng.spec_k == 3
    assert eng.generate([ids], sp)[0] == truth
    assert eng.stats["spec_rounds"] > 0 and eng.stats["spec_drafted"] == 3 * eng.stats["spec_rounds"]
    # drafts that are right (taken from the known continuation) are accepted: fewer rounds than tokens
    eng = LLMEngine(model, EngineOptions(max_ctx=512, max_batch_tokens=64, max_seqs=2, spec_k=3))
    seq = eng.add_request(ids, sp)
    real = head.draft
    seen = []

    def oracle(h, tok, k, ctx):
        seen.append((int(ctx["pos"]), tuple(ctx["block_table"].shape)))
        g = len(seq.tokens) - len(ids)
        real(h, tok, 1, ctx)                         # the real head still runs on the live cache and position
        return (list(truth[g:g + k]) + [0] * k)[:k]
    head.draft = oracle
    try:
        while not seq.finished:
            eng.step()
    finally:
        head.draft = real
    assert seq.tokens[len(ids):] == truth
    assert eng.stats["spec_accepted"] > 0 and eng.stats["spec_rounds"] < len(truth)
    assert seen[0][0] == len(ids) and all(b[0] == 1 for _, b in seen)
    # a head of another width or vocabulary is refused
    bad = synth_assistant_config(dataclasses.replace(cfg, hidden=128), n_layers=2)
    bpath = str(tmp_path / "bad.gguf")
    write_synthetic_assistant_gguf(bad, bpath)
    with pytest.raises(ValueError):
        load_assistant_head(model, bpath)
