"""int8 KV cache (per-row scales): storage rule, attention over it, block copies and the engine option, on the CPU path."""
import torch

from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.models import build_model
from machx_inference_engine_b200.models.transformer import KVCache
from machx_inference_engine_b200.ops import ref
from machx_inference_engine_b200.runtime.engine import EngineOptions, LLMEngine, SamplingParams


def test_rows_are_symmetric_int8_with_max_over_127_scale():
    T, n_q, n_kv, hd = 9, 4, 2, 64
    torch.manual_seed(0)
    qkv = (torch.randn(T, (n_q + 2 * n_kv) * hd) * 2).to(torch.bfloat16)
    slots = torch.arange(T, dtype=torch.int64) + 3
    c8 = KVCache(1, 2, n_kv, hd, torch.device("cpu"), dtype="int8")
    c16 = KVCache(1, 2, n_kv, hd, torch.device("cpu"))
    pos = torch.zeros(T, dtype=torch.int32)
    ref.qkv_post(qkv, None, None, None, pos, None, None, slots, c8.k[0], c8.v[0], n_q, n_kv, hd, 0, kv_scales=c8.scales(0))
    ref.qkv_post(qkv, None, None, None, pos, None, None, slots, c16.k[0], c16.v[0], n_q, n_kv, hd, 0)
    assert c8.k[0].dtype == torch.int8 and c16.scales(0) is None
    for q8, sc, full in ((c8.k[0], c8.ks[0], c16.k[0]), (c8.v[0], c8.vs[0], c16.v[0])):
        rows = full.float()[0, :, 3:3 + T]
        assert torch.allclose(sc[0, :, 3:3 + T], rows.abs().amax(-1) / 127.0, rtol=1e-2)
        assert int(q8[0, :, 3:3 + T].abs().max()) == 127
        deq = q8.float() * sc.unsqueeze(-1)
        assert float((deq - full.float()).abs().max()) <= float(sc.max()) * 0.51 + 0.02
    assert KVCache.bytes_per_block(4, 2, 64, "int8") * 2 < KVCache.bytes_per_block(4, 2, 64) * 1.1


def test_copy_blocks_moves_scales_too():
    c = KVCache(2, 4, 1, 64, torch.device("cpu"), dtype="int8")
    for l in (0, 1):
        c.k[l][1].fill_(7); c.ks[l][1].fill_(0.5); c.v[l][1].fill_(-3); c.vs[l][1].fill_(0.25)
    c.copy_blocks([1], [3])
    for l in (0, 1):
        assert bool((c.k[l][3] == 7).all()) and bool((c.ks[l][3] == 0.5).all()) and bool((c.vs[l][3] == 0.25).all())


def test_engine_with_int8_cache_tracks_the_bf16_engine():
    cfg = preset("tiny-qwen3")
    torch.manual_seed(0)
    m = build_model(cfg, torch.device("cpu"), quant="q8_0", max_ctx=1024)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab, (300,), generator=g).tolist()
    logits = {}
    for dt in ("bf16", "int8"):
        eng = LLMEngine(m, EngineOptions(max_ctx=1024, max_batch_tokens=128, max_seqs=2, kv_dtype=dt))
        assert eng.kv.dtype == dt
        grabbed = []
        fwd = m.forward

        def grab(fb, *a, **k):
            out = fwd(fb, *a, **k)
            grabbed.append(out.float())
            return out
        m.forward = grab
        try:
            seq = eng.add_request(ids, SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))
            while not seq.finished:
                eng.step()
        finally:
            m.forward = fwd
        logits[dt] = torch.cat([x[-1:] for x in grabbed])        # last row of every prefill chunk and decode step
        # a second request with the same prompt reuses the quantised prefix blocks
        seq2 = eng.add_request(ids, SamplingParams(max_tokens=2, temperature=0.0, ignore_eos=True))
        while not seq2.finished:
            eng.step()
        assert seq2.tokens[len(ids):len(ids) + 2] == seq.tokens[len(ids):len(ids) + 2]
    cos = torch.nn.functional.cosine_similarity(logits["bf16"], logits["int8"], dim=1)
    assert float(cos.min()) > 0.995
