"""The row-sharded prefill path (csrc/cuda/shard.cu, parallel/sharded.py) on one GPU with a world of one rank: every kernel of
the path runs (norm with gather stores, the GEMM that waits for gather flags, reduce-scatter epilogue and its consumer, expert
dispatch plan / send / finalize, return and combine), with this rank as its own and only peer, so no kernel ever waits for
another launch.  The multi-rank form of the same path is checked against one GPU in tests/test_parallel.py."""
import pytest
import torch

from machx_inference_engine_b200.formats.model_config import preset
from machx_inference_engine_b200.models import build_model
from machx_inference_engine_b200.ops import ref
from machx_inference_engine_b200.parallel.comm import ParallelCtx

pytestmark = pytest.mark.gpu


def _cos(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))


def _prefill(model, ids, n_blocks):
    from machx_inference_engine_b200.models.transformer import KV_BLOCK, ForwardBatch
    d = model.device
    T = len(ids)
    kv = model.new_kv_cache(n_blocks + 2)
    pos = torch.arange(T, dtype=torch.int32, device=d)
    bt = torch.arange(1, n_blocks + 1, dtype=torch.int32, device=d).unsqueeze(0)
    slot = bt[0][(pos // KV_BLOCK).long()].long() * KV_BLOCK + (pos % KV_BLOCK).long()
    fb = ForwardBatch(torch.tensor(ids, dtype=torch.int32, device=d), pos, slot, bt, torch.tensor([T], dtype=torch.int32, device=d),
                      torch.tensor([0, T], dtype=torch.int32, device=d), T, logit_rows=torch.arange(T, device=d))
    return model.forward(fb, kv).float()


@pytest.mark.parametrize("name,quant", [("tiny-gpt-oss", "mxfp4"), ("tiny-llama", "q8_0")])
def test_sharded_prefill_equals_the_replicated_path_on_one_rank(name, quant):
    from machx_inference_engine_b200.ops import cuda as K
    from machx_inference_engine_b200.parallel.fused import FusedComm
    from machx_inference_engine_b200.parallel.sharded import attach
    dev = torch.device("cuda:0")
    cfg = preset(name)
    par = ParallelCtx()
    model = build_model(cfg, dev, par, quant=quant, max_ctx=1024, gen_device="cpu")
    ids = torch.randint(0, cfg.vocab, (640,), generator=torch.Generator().manual_seed(3)).tolist()
    want = _prefill(model, ids, 5)
    par.fused = FusedComm.create(par, dev, max_tokens=1024, max_width=4096)
    sc = attach(par, dev, cfg, 1024, force=True)
    try:
        assert sc is not None and model._can_shard(type("FB", (), {"T": 640, "want_hidden": False})(), None)
        got = _prefill(model, ids, 5)
        got2 = _prefill(model, ids, 5)
        K.check_status()
    finally:
        par.sharded = None
        par.fused.close()
        par.fused = None
        sc.close()
    assert torch.equal(got, got2)                                   # fixed summation orders: run to run identical
    # The two paths round the output projection differently (bias added before / after the bf16 rounding of the partial); with
    # MXFP8 expert inputs such one-step differences flip a fraction of the e4m3 roundings (see test_gpu_models.py)
    moe = "gpt-oss" in name
    assert _cos(got, want) > (0.997 if moe else 0.9995)
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > (0.93 if moe else 0.97)


def test_dispatch_plan_is_the_stable_counting_sort_of_the_packer():
    """With one rank the dispatch plan must place every (token, slot) pair where the single-GPU packer places it, build the same
    tile table, and the receive buffer must hold the rows the single-GPU quantiser writes."""
    from machx_inference_engine_b200.ops import cuda as K
    from machx_inference_engine_b200.parallel.sharded import ShardedComm
    dev = torch.device("cuda:0")
    torch.manual_seed(5)
    R, H, E, topk = 384, 512, 16, 4
    sc = ShardedComm(ParallelCtx(), dev, H, 512, n_experts=E, top_k=topk)
    try:
        h = torch.randn(R, H, device=dev).to(torch.bfloat16)
        logits = torch.randn(R, E, device=dev)
        logits[:, 3] += 3.0                                        # one expert with several tiles
        logits[:, 7] -= 50.0                                       # one with none
        idx, w = K.moe_route(logits, None, topk)
        xq, sfx, plan = sc.dispatch(h, idx)
        pk = ref.moe_pack(idx, E)
        nt = int(pk.num_tiles[0])
        assert torch.equal(plan.num_tiles.cpu(), pk.num_tiles.cpu())
        assert torch.equal(plan.pair_pos, pk.pair_to_packed)
        assert torch.equal(plan.tile_expert[:nt], pk.tile_expert[:nt]) and torch.equal(plan.tile_valid[:nt], pk.tile_valid[:nt])
        xq_ref, sfx_ref = K.moe_quant(h, pk.max_rows, sc.max_tiles, 128, src_index=pk.packed_token, row_limit=pk.num_tiles)
        live = pk.packed_token[: int(pk.num_tiles[1])] >= 0
        assert torch.equal(xq[: live.numel()][live], xq_ref[: live.numel()][live])
        # scale atoms: compare the bytes of live rows only (pad rows are never read)
        rows = live.nonzero().flatten()
        tile, r = rows // 128, rows % 128
        off = (r % 32) * 16 + (r // 32) * 4
        for kb in range(sfx.shape[0]):
            for q in range(4):
                assert torch.equal(sfx[kb, tile, off + q], sfx_ref[kb, tile, off + q])
        # round trip: identity experts -> combine returns sum_k w * row
        y = torch.zeros(sc.p_max, H, dtype=torch.bfloat16, device=dev)
        y[plan.pair_pos.long()] = h.repeat_interleave(topk, dim=0)
        out = sc.combine(y, plan, w)
        K.check_status()
        assert torch.allclose(out, h.float() * w.sum(dim=1, keepdim=True), rtol=1e-2, atol=1e-2)
    finally:
        sc.close()


def test_a_flag_that_nobody_sets_ends_the_wait_with_a_status_and_leaves_the_gpu_usable():
    """Failure detection on the device without a fault: consumers wait for their peers' flags with a time limit.  Here the
    expected sequence number is raised by hand, so the flag this (only) rank waits for never arrives; with the limit lowered to a
    few milliseconds the kernels return, the status word reports the peer-flag code, and the next ordinary launch works."""
    import ctypes as C
    from machx_inference_engine_b200 import _lib
    from machx_inference_engine_b200.ops import cuda as K
    from machx_inference_engine_b200.parallel.fused import FusedComm, ReducedDelta
    from machx_inference_engine_b200.parallel.sharded import ShardedComm
    dev = torch.device("cuda:0")
    par = ParallelCtx()
    R, H, topk = 128, 256, 2
    # (1) the sharded path's combine: limit 2^22 cycles (about 2 ms)
    sc = ShardedComm(par, dev, H, 128, n_experts=4, top_k=topk, wait_cycles_log2=22)
    try:
        sc.seq[3] += 1                                   # FL_RET: expect a return that no kernel will publish
        w = torch.full((R, topk), 0.5, device=dev)
        out = torch.empty(R, H, dtype=torch.float32, device=dev)
        K._check(_lib.cuda().mx_moe_combine_wait(sc._ws_ref, K._p(w), K._p(out), R, H, topk, K._stream()), "moe_combine_wait")
        with pytest.raises(K.KernelError, match="peer flag"):
            K.check_status()
    finally:
        sc.close()
    # (2) the fused all-reduce's consumer (residual add + RMSNorm over the inbox): same, through the library-wide limit
    lib = _lib.cuda()
    assert lib.mx_set_wait_limit_cycles(C.c_longlong(1 << 22)) == 0
    fc = FusedComm.create(par, dev, max_tokens=128, max_width=H)
    try:
        fc.seq += 1                                      # a partial that no producer has pushed
        x = torch.randn(8, H, device=dev)
        with pytest.raises(K.KernelError, match="peer flag"):
            fc.rmsnorm(x, torch.ones(H, device=dev), 1e-5, ReducedDelta(fc, 8, H, bf16=False))
            K.check_status()
    finally:
        assert lib.mx_set_wait_limit_cycles(C.c_longlong(2000000000)) == 0
        fc.close()
    # the context is intact: an ordinary kernel runs and is correct
    x = torch.randn(4, H, device=dev)
    got = K.rmsnorm(x, torch.ones(H, device=dev), 1e-5)
    K.check_status()
    want = ref.rmsnorm(x.clone(), torch.ones(H, device=dev), 1e-5)
    assert torch.allclose(got.float(), want.float(), atol=2e-2)
