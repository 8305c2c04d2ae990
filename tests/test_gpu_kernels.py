"""Numerics of every sm_100a kernel against the PyTorch fp32 oracle (ops.ref), small and ragged shapes.

Mirrors the reference's per-kernel unit tests (tests/unit/*.cpp: attention_test, moe_test,
gemv_q4k_test, mxfp4_dequant_test, sampler_test, elementwise_test) with the host scalar
references replaced by ops.ref.
"""
import math

import pytest
import torch

from machx_inference_engine_b200.ops import ref
from machx_inference_engine_b200.ops.weights import WFormat, from_dense

pytestmark = pytest.mark.gpu

FMTS = [WFormat.BF16, WFormat.Q8, WFormat.Q4K, WFormat.Q6K, WFormat.MXFP4]


def K():
    from machx_inference_engine_b200.ops import cuda
    return cuda


def dev():
    return torch.device("cuda:0")


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def make_weight(fmt, N, Kd, E=1, seed=0, scale=0.05):
    g = torch.Generator(device="cpu").manual_seed(seed)
    w = torch.randn(E, N, Kd, generator=g) * scale
    return from_dense(w, fmt).to(dev())


@pytest.mark.parametrize("fmt", FMTS)
def test_dequant_layouts_roundtrip(fmt):
    # the runtime layout decodes (on the GPU through embed) to what the torch decoder says
    qw = make_weight(fmt, 64, 512)
    ids = torch.arange(64, dtype=torch.int32, device=dev())
    got = K().embed(qw, ids)
    want = qw.dequantize()[0]
    assert torch.allclose(got, want, rtol=0, atol=1e-6 * float(want.abs().max()) + 1e-7), rel_err(got, want)


def test_e2m1_decoders_bit_exact():
    # both in-kernel E2M1 decoders (byte-permute tables -> bf16, hardware cvt -> fp16) against the code table,
    # for every byte value in every byte lane (the reference checks its decoder the same way: tests/mxfp4_dequant_test.cpp)
    import ctypes as C
    from machx_inference_engine_b200 import _lib
    vals = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6])
    words = torch.randint(0, 2 ** 31 - 1, (4096,), dtype=torch.int64)
    words[:256] = torch.arange(256) * 0x01010101 % (2 ** 32)
    w32 = words.to(torch.int64).to(dev())
    inp = (w32 & 0xFFFFFFFF).to(torch.int64)
    packed = torch.empty(4096, dtype=torch.int32, device=dev())
    packed.copy_(torch.where(inp >= 2 ** 31, inp - 2 ** 32, inp).to(torch.int32))
    out = torch.empty(4096, 16, device=dev())
    rc = _lib.cuda().mx_e2m1_probe(C.c_void_p(packed.data_ptr()), C.c_void_p(out.data_ptr()), 4096, C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    codes = torch.stack([(inp >> (4 * j)) & 15 for j in range(8)], dim=1).cpu()
    want = vals[codes]
    got = out.cpu()
    assert torch.equal(got[:, :8], want), "byte-permute decoder"
    assert torch.equal(got[:, 8:], want), "hardware cvt decoder"


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M", [1, 3, 8])
def test_gemv(fmt, M):
    N, Kd = 200, 768            # N not a multiple of the 16 rows per CTA
    qw = make_weight(fmt, N, Kd)
    x = (torch.randn(M, Kd, device=dev()) * 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device=dev())
    got = K().linear(x, qw, bias=bias, out_f32=True)
    want = ref.linear(x, qw, bias=bias, out_f32=True)
    assert rel_err(got, want) < 2e-3


@pytest.mark.parametrize("fmt", [WFormat.BF16, WFormat.MXFP4, WFormat.Q4K, WFormat.Q8])
def test_gemv_gated(fmt):
    F, Kd = 96, 512
    qw = make_weight(fmt, 2 * F, Kd)
    x = (torch.randn(2, Kd, device=dev())).to(torch.bfloat16)
    bias = torch.randn(2 * F, device=dev()) * 0.1
    for act in (ref.ACT_SWIGLU, ref.ACT_SWIGLU_OAI, ref.ACT_GEGLU):
        got = K().linear(x, qw, bias=bias, act=act, out_f32=True)
        want = ref.linear(x, qw, bias=bias, act=act, out_f32=True)
        assert rel_err(got, want) < 3e-3, act


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("shape", [(128, 128, 256), (200, 328, 512), (1000, 2880, 2816)])
def test_gemm_tcgen05(fmt, shape):
    M, N, Kd = shape
    if fmt in (WFormat.Q4K, WFormat.Q6K) and Kd % 256:
        pytest.skip("super-block formats need K % 256 == 0")
    qw = make_weight(fmt, N, Kd)
    x = (torch.randn(M, Kd, device=dev()) * 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device=dev())
    for bn in (128, 64, 32):
        got = K().gemm(x, qw, bias=bias, out_f32=True, bn=bn)
        K().check_status()
        want = ref.linear(x, qw, bias=bias, out_f32=True)
        # weights pass through bf16 inside the tensor-core path
        assert rel_err(got, want) < 6e-3, (bn, rel_err(got, want))


@pytest.mark.parametrize("fmt", [WFormat.Q8, WFormat.Q4K, WFormat.Q6K, WFormat.MXFP4])
def test_linear_long_chunk_decodes_the_weight_once(fmt):
    """From DEQUANT_ONCE_MIN_M rows on `linear` decodes a quantised dense weight to bf16 once and runs the TMA-fed kernel: the same values as
    the in-kernel decode (both multiply bf16 weights), with and without a gated epilogue."""
    M, N, Kd = 1100, 640, 1024
    assert M >= K().DEQUANT_ONCE_MIN_M
    qw = make_weight(fmt, N, Kd)
    x = (torch.randn(M, Kd, device=dev()) * 0.5).to(torch.bfloat16)
    bias = torch.randn(N, device=dev())
    got = K().linear(x, qw, bias=bias, out_f32=True)
    K().check_status()
    assert rel_err(got, ref.linear(x, qw, bias=bias, out_f32=True)) < 6e-3
    assert rel_err(got, K().gemm(x, qw, bias=bias, out_f32=True)) < 1e-3
    got = K().linear(x, qw, act=ref.ACT_SWIGLU)
    assert rel_err(got, K().gemm(x, qw, act=ref.ACT_SWIGLU)) < 2e-3
    # below the threshold nothing changes: same kernel as `gemm`
    n = K().DEQUANT_ONCE_MIN_M - 16
    assert n > 8 and torch.equal(K().linear(x[:n].contiguous(), qw, bias=bias, out_f32=True), K().gemm(x[:n].contiguous(), qw, bias=bias, out_f32=True))


def test_gemm_ragged_k_and_bf16_out():
    M, N, Kd = 130, 72, 2880      # K = 45 * 64, N not a multiple of 32
    qw = make_weight(WFormat.MXFP4, N, Kd)
    x = (torch.randn(M, Kd, device=dev()) * 0.5).to(torch.bfloat16)
    got = K().gemm(x, qw)
    want = ref.linear(x, qw)
    assert got.dtype == torch.bfloat16 and rel_err(got, want) < 1e-2
    qw = make_weight(WFormat.BF16, N, 2888)     # K % 64 == 8: TMA zero fill on the last k tile
    x = (torch.randn(M, 2888, device=dev()) * 0.5).to(torch.bfloat16)
    assert rel_err(K().gemm(x, qw, out_f32=True), ref.linear(x, qw, out_f32=True)) < 6e-3


@pytest.mark.parametrize("act", [ref.ACT_SWIGLU, ref.ACT_SWIGLU_OAI, ref.ACT_GEGLU])
def test_gemm_gated_epilogue(act):
    M, F, Kd = 300, 160, 512
    qw = make_weight(WFormat.MXFP4, 2 * F, Kd)
    x = (torch.randn(M, Kd, device=dev())).to(torch.bfloat16)
    bias = torch.randn(2 * F, device=dev()) * 0.1
    got = K().gemm(x, qw, bias=bias, act=act, out_f32=True)
    want = ref.linear(x, qw, bias=bias, act=act, out_f32=True)
    assert rel_err(got, want) < 1e-2


@pytest.mark.parametrize("fmt", [WFormat.MXFP4, WFormat.Q8, WFormat.BF16])
def test_grouped_gemm_and_moe_pipeline(fmt):
    T, H, F, E, topk = 300, 256, 128, 8, 2
    torch.manual_seed(1)
    x = (torch.randn(T, H, device=dev())).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev())
    rb = torch.randn(E, device=dev()) * 0.1
    idx, w = K().moe_route(logits, rb, topk)
    idx_r, w_r = ref.moe_route(logits, rb, topk)
    assert torch.equal(idx, idx_r) and torch.allclose(w, w_r, atol=1e-5)
    pk = K().moe_pack(idx, E)
    pk_r = ref.moe_pack(idx, E)
    assert torch.equal(pk.num_tiles, pk_r.num_tiles)
    nrows = int(pk.num_tiles[1])
    assert torch.equal(pk.packed_token[:nrows], pk_r.packed_token[:nrows])
    assert torch.equal(pk.pair_to_packed, pk_r.pair_to_packed)
    assert torch.equal(pk.tile_expert[: int(pk.num_tiles[0])], pk_r.tile_expert[: int(pk.num_tiles[0])])
    xp = K().moe_gather(x, pk, zero_pad=True)
    assert torch.equal(xp[:nrows], ref.moe_gather(x, pk_r)[:nrows])
    live = pk_r.packed_token[:nrows] >= 0                               # default: padding rows are left unwritten
    assert torch.equal(K().moe_gather(x, pk)[:nrows][live], ref.moe_gather(x, pk_r)[:nrows][live])
    gu = make_weight(fmt, 2 * F, H, E=E, seed=3)
    dn = make_weight(fmt, H, F, E=E, seed=4)
    gb = torch.randn(E, 2 * F, device=dev()) * 0.1
    db = torch.randn(E, H, device=dev()) * 0.1
    h = K().grouped_linear(xp, gu, pk.tile_expert, pk.num_tiles, bias=gb, act=ref.ACT_SWIGLU_OAI)
    h_r = ref.grouped_linear(xp, gu, pk_r.tile_expert, pk_r.num_tiles, bias=gb, act=ref.ACT_SWIGLU_OAI)
    live = pk.packed_token[:nrows] >= 0
    assert rel_err(h[:nrows][live], h_r[:nrows][live]) < 1.5e-2
    y = K().grouped_linear(h, dn, pk.tile_expert, pk.num_tiles, bias=db)
    y_r = ref.grouped_linear(h_r, dn, pk_r.tile_expert, pk_r.num_tiles, bias=db)
    out = K().moe_combine(y, pk, w)
    out_r = ref.moe_combine(y_r, pk_r, w_r)
    assert rel_err(out, out_r) < 2e-2
    # expert-parallel packing: only experts [2,5) are owned
    pk2, pk2_r = K().moe_pack(idx, E, 2, 5), ref.moe_pack(idx, E, 2, 5)
    assert torch.equal(pk2.pair_to_packed, pk2_r.pair_to_packed) and torch.equal(pk2.num_tiles, pk2_r.num_tiles)


def test_expert_gemv():
    H, F, E = 512, 64, 8
    gu = make_weight(WFormat.MXFP4, 2 * F, H, E=E, seed=5)
    dn = make_weight(WFormat.MXFP4, H, F, E=E, seed=6)
    x = torch.randn(2, H, device=dev()).to(torch.bfloat16)
    slot_e = torch.tensor([1, 7, 3, 0, 2, 2, 5, 4], dtype=torch.int32, device=dev())   # 2 tokens x 4 slots
    gb = torch.randn(E, 2 * F, device=dev()) * 0.1
    h = K().expert_gemv(x, gu, slot_e, x_div=4, bias=gb, act=ref.ACT_SWIGLU_OAI)
    h_r = ref.expert_gemv(x, gu, slot_e, x_div=4, bias=gb, act=ref.ACT_SWIGLU_OAI)
    assert rel_err(h, h_r) < 1e-2
    sc = torch.rand(8, device=dev())
    y = K().expert_gemv(h, dn, slot_e, x_div=1, slot_scale=sc, out_f32=True)
    y_r = ref.expert_gemv(h, dn, slot_e, x_div=1, slot_scale=sc, out_f32=True)
    assert rel_err(y, y_r) < 5e-3


@pytest.mark.parametrize("fmt", [WFormat.BF16, WFormat.Q8, WFormat.MXFP4])
def test_streaming_gemv_matches_register_gemv_and_oracle(fmt):
    """The bulk-copy streaming kernel and the register-streamed kernel are two implementations of one contract."""
    k = K()
    for (M, N, Kd) in [(1, 2880, 2880), (1, 200, 4096), (3, 515, 1024), (8, 96, 2880), (1, 64, 14336)]:
        if fmt == WFormat.MXFP4 and M > 1:
            continue
        w = make_weight(fmt, N, Kd, seed=N)
        x = (torch.randn(M, Kd, device=dev()) * 3).to(torch.bfloat16)
        bias = torch.randn(N, device=dev())
        want = ref.linear(x, w, bias=bias, out_f32=True)
        k.set_gemv_path("stream")
        a = k.linear(x, w, bias=bias, out_f32=True)
        k.set_gemv_path("register")
        b = k.linear(x, w, bias=bias, out_f32=True)
        k.set_gemv_path("auto")
        k.check_status()
        assert rel_err(a, want) < 4e-3, (M, N, Kd)
        assert rel_err(b, want) < 4e-3, (M, N, Kd)
    if fmt == WFormat.Q8:
        # gated epilogue of the dp4a form: whole rows (K <= 3072) and K chunks with both planes copied per row
        for (M, F, Kd) in [(1, 96, 2880), (2, 208, 4096), (1, 64, 14336)]:       # (F a multiple of 16)
            w = make_weight(fmt, 2 * F, Kd, seed=F)
            x = torch.randn(M, Kd, device=dev()).to(torch.bfloat16)
            bias = torch.randn(2 * F, device=dev()) * 0.1
            k.set_gemv_path("stream")
            got = k.linear(x, w, bias=bias, act=ref.ACT_SWIGLU, out_f32=True)
            k.set_gemv_path("auto")
            k.check_status()
            assert rel_err(got, ref.linear(x, w, bias=bias, act=ref.ACT_SWIGLU, out_f32=True)) < 3e-3, (M, F, Kd)
    # activations with a large dynamic range (fp16 staging of the MXFP4 path must not overflow or flush them)
    # (and the block-scaled 16-bit staging of the Q8 path must keep small elements beside large ones)
    if fmt in (WFormat.MXFP4, WFormat.Q8):
        w = make_weight(fmt, 256, 2880, seed=5)
        x = torch.randn(1, 2880, device=dev())
        x[0, ::97] *= 3000.0
        x[0, 1::2] *= 1e-3
        x = x.to(torch.bfloat16)
        k.set_gemv_path("stream")
        got = k.linear(x, w, out_f32=True)
        k.set_gemv_path("auto")
        assert rel_err(got, ref.linear(x, w, out_f32=True)) < 4e-3


@pytest.mark.parametrize("fmt", [WFormat.Q4K, WFormat.Q6K])
def test_streaming_gemv_kquants(fmt):
    """Q4_K / Q6_K through the bulk-copy streaming kernel (the codes against block-scaled 16-bit activations in dp4a): plain rows
    with one and several activation rows, a K that is split into chunks, the gated epilogue (Q4_K), activations with outliers."""
    k = K()
    try:
        for (M, N, Kd) in [(1, 200, 4096), (1, 520, 1024), (3, 515, 1024), (8, 96, 2048), (1, 64, 14336), (2, 40, 14336), (1, 128, 5120), (1, 72, 17408), (1, 40, 1280)]:
            w = make_weight(fmt, N, Kd, seed=N)
            x = (torch.randn(M, Kd, device=dev()) * 3).to(torch.bfloat16)
            bias = torch.randn(N, device=dev())
            want = ref.linear(x, w, bias=bias, out_f32=True)
            k.set_gemv_path("stream")
            a = k.linear(x, w, bias=bias, out_f32=True)
            k.set_gemv_path("register")
            b = k.linear(x, w, bias=bias, out_f32=True)
            k.check_status()
            assert rel_err(a, want) < 1e-3, (M, N, Kd)
            assert rel_err(b, want) < 4e-3, (M, N, Kd)
        for (M, F, Kd) in [(1, 96, 1024), (2, 400, 4096), (1, 64, 6144)] if fmt == WFormat.Q4K else []:
            w = make_weight(WFormat.Q4K, 2 * F, Kd, seed=F)
            x = torch.randn(M, Kd, device=dev()).to(torch.bfloat16)
            bias = torch.randn(2 * F, device=dev()) * 0.1
            k.set_gemv_path("stream")
            for act in (ref.ACT_SWIGLU, ref.ACT_GEGLU):
                got = k.linear(x, w, bias=bias, act=act, out_f32=True)
                assert rel_err(got, ref.linear(x, w, bias=bias, act=act, out_f32=True)) < 3e-3, (M, F, Kd, act)
        w = make_weight(fmt, 256, 4096, seed=5)
        x = torch.randn(1, 4096, device=dev())
        x[0, ::97] *= 3000.0
        x[0, 1::2] *= 1e-3
        x[0, 512:768] = 0
        x = x.to(torch.bfloat16)
        k.set_gemv_path("stream")
        assert rel_err(k.linear(x, w, out_f32=True), ref.linear(x, w, out_f32=True)) < 1e-3
        k.check_status()
    finally:
        k.set_gemv_path("auto")


def test_streaming_gemv_bf16_eight_warps():
    """The optional bf16 configuration with eight consumer warps per CTA gives the same numbers as the default one."""
    k = K()
    try:
        for (M, N, Kd) in [(1, 2880, 2880), (2, 200, 4096), (1, 64, 14336)]:
            w = make_weight(WFormat.BF16, N, Kd, seed=N)
            x = torch.randn(M, Kd, device=dev()).to(torch.bfloat16)
            outs = []
            for wide in (False, True):
                k.set_gemv_bf16_wide(wide)
                outs.append(k.linear(x, w, out_f32=True))
            k.check_status()
            assert torch.equal(outs[0], outs[1]), (M, N, Kd)
    finally:
        k.set_gemv_bf16_wide(False)


def test_streaming_gemv_chunk_copies_both_ways():
    """Chunked rows arrive by tiled TMA loads (default) or by one bulk copy per row: the same numbers either way, for every chunked
    format, plain and gated, with a last row block that is cut by the matrix edge."""
    k = K()
    try:
        k.set_gemv_path("stream")
        for fmt, N, Kd, act in [(WFormat.Q4K, 200, 4096, ref.ACT_NONE), (WFormat.Q4K, 2 * 208, 6144, ref.ACT_SWIGLU), (WFormat.Q6K, 72, 14336, ref.ACT_NONE),
                                (WFormat.Q8, 100, 14336, ref.ACT_NONE), (WFormat.Q8, 2 * 112, 4096, ref.ACT_SWIGLU), (WFormat.Q4K, 40, 5120, ref.ACT_NONE)]:
            w = make_weight(fmt, N, Kd, seed=N)
            x = torch.randn(1, Kd, device=dev()).to(torch.bfloat16)
            outs = []
            for tma in (True, False):
                k.set_gemv_tma(tma)
                outs.append(k.linear(x, w, act=act, out_f32=True))
            k.check_status()
            assert torch.equal(outs[0], outs[1]), (fmt, N, Kd)
            assert rel_err(outs[0], ref.linear(x, w, act=act, out_f32=True)) < 3e-3, (fmt, N, Kd)
    finally:
        k.set_gemv_tma(True)
        k.set_gemv_path("auto")


@pytest.mark.parametrize("fmt,H", [(WFormat.MXFP4, 512), (WFormat.Q8, 512), (WFormat.Q4K, 512), (WFormat.Q8, 4096), (WFormat.Q4K, 4096)])
def test_streaming_expert_gemv_with_foreign_experts(fmt, H):
    # H = 4096: the gate|up rows are cut into K chunks, fetched by tiled loads whose row coordinate carries the expert's offset
    k = K()
    E, F, topk = 8, 256, 4
    gu = make_weight(fmt, 2 * F, H, E=E, seed=1)
    dn = make_weight(fmt, H, F, E=E, seed=2)
    gub, dnb = torch.randn(E, 2 * F, device=dev()), torch.randn(E, H, device=dev())
    x = torch.randn(2, H, device=dev()).to(torch.bfloat16)
    se = torch.tensor([1, 6, 2, 7, 0, 3, 5, 2], dtype=torch.int32, device=dev())
    for path, (e_lo, e_hi) in [("stream", (0, 8)), ("stream", (2, 6)), ("auto", (2, 6))]:
        k.set_gemv_path(path)
        g, d = gu.slice_experts(e_lo, e_hi), dn.slice_experts(e_lo, e_hi)
        gb, db = gub[e_lo:e_hi].contiguous(), dnb[e_lo:e_hi].contiguous()
        a = k.expert_gemv(x, g, se, x_div=topk, bias=gb, act=ref.ACT_SWIGLU_OAI, e_lo=e_lo)
        want = ref.expert_gemv(x, g, se, x_div=topk, bias=gb, act=ref.ACT_SWIGLU_OAI, e_lo=e_lo)
        assert rel_err(a, want) < 1e-2
        y = k.expert_gemv(want, d, se, x_div=1, bias=db, e_lo=e_lo, out_f32=True)
        assert rel_err(y, ref.expert_gemv(want, d, se, x_div=1, bias=db, e_lo=e_lo, out_f32=True)) < 5e-3
        foreign = [i for i, e in enumerate(se.tolist()) if not (e_lo <= e < e_hi)]
        assert all(float(y[i].abs().max()) == 0.0 for i in foreign)
    k.set_gemv_path("auto")
    k.check_status()


@pytest.mark.parametrize("E,K_top,T,rng", [(128, 4, 2048, (0, 128)), (512, 10, 700, (0, 512)), (8, 2, 5, (2, 6)), (32, 4, 1, (0, 32))])
def test_moe_pack_is_a_stable_counting_sort(E, K_top, T, rng):
    g = torch.Generator().manual_seed(E + T)
    idx = torch.stack([torch.randperm(E, generator=g)[:K_top] for _ in range(T)]).to(torch.int32).to(dev())
    got = K().moe_pack(idx, E, rng[0], rng[1])
    want = ref.moe_pack(idx.cpu(), E, rng[0], rng[1])
    assert int(got.num_tiles[0]) == int(want.num_tiles[0]) and int(got.num_tiles[1]) == int(want.num_tiles[1])
    rows = int(want.num_tiles[1])
    assert torch.equal(got.packed_token[:rows].cpu(), want.packed_token[:rows])
    assert torch.equal(got.pair_to_packed.cpu(), want.pair_to_packed)
    assert torch.equal(got.tile_expert[:int(want.num_tiles[0])].cpu(), want.tile_expert[:int(want.num_tiles[0])])


@pytest.mark.parametrize("fmt", [WFormat.MXFP4, WFormat.Q8, WFormat.Q4K])
def test_expert_group_gemv_batched_decode(fmt):
    """Compact packing + expert-major GEMV (the MoE path for decode batches of 9..512 tokens) against the oracle, including an
    expert with more than eight rows (two passes), empty experts and an expert-parallel shard."""
    k = K()
    E, H, F, topk, T = 16, 512, 256, 4, 40
    gu = make_weight(fmt, 2 * F, H, E=E, seed=3)
    dn = make_weight(fmt, H, F, E=E, seed=4)
    gub, dnb = torch.randn(E, 2 * F, device=dev()), torch.randn(E, H, device=dev())
    g = torch.Generator().manual_seed(9)
    idx = torch.stack([torch.randperm(E - 3, generator=g)[:topk] for _ in range(T)]).to(torch.int32)     # experts 13..15 stay empty
    idx[:20, 0] = 2                                                                                      # expert 2 gets >= 20 rows
    idx[:20, 1:] = torch.stack([torch.randperm(E - 4, generator=g)[:topk - 1] + 3 for _ in range(20)]).to(torch.int32)
    idx = idx.to(dev())
    x = torch.randn(T, H, device=dev()).to(torch.bfloat16)
    for e_lo, e_hi in [(0, E), (0, 8)]:
        pk = k.moe_pack(idx, E, e_lo, e_hi, tile=1)
        pk_ref = ref.moe_pack(idx.cpu(), E, e_lo, e_hi, tile=1)
        n_rows = int(pk_ref.num_tiles[1])
        assert torch.equal(pk.pair_to_packed.cpu(), pk_ref.pair_to_packed) and torch.equal(pk.packed_token[:n_rows].cpu(), pk_ref.packed_token[:n_rows])
        gs, ds = gu.slice_experts(e_lo, e_hi), dn.slice_experts(e_lo, e_hi)
        gb, db = gub[e_lo:e_hi].contiguous(), dnb[e_lo:e_hi].contiguous()
        a = k.expert_group_gemv(x, gs, pk, x_index=pk.packed_token, bias=gb, act=ref.ACT_SWIGLU_OAI, e_lo=e_lo)
        a_ref = ref.expert_group_gemv(x, gs, pk, x_index=pk.packed_token, bias=gb, act=ref.ACT_SWIGLU_OAI, e_lo=e_lo)
        assert rel_err(a[:n_rows], a_ref[:n_rows]) < 1e-2
        y = k.expert_group_gemv(a_ref, ds, pk, bias=db, e_lo=e_lo)
        y_ref = ref.expert_group_gemv(a_ref, ds, pk, bias=db, e_lo=e_lo)
        assert rel_err(y[:n_rows], y_ref[:n_rows]) < 1e-2
        w = torch.rand(T, topk, device=dev())
        assert rel_err(k.moe_combine(y_ref, pk, w), ref.moe_combine(y_ref, pk, w)) < 1e-3
    k.check_status()


def test_rmsnorm_residual_and_saturation():
    T, H = 37, 2880
    x = torch.randn(T, H, device=dev()) * 3
    x[0, :8] = 70000.0           # beyond fp16 range: the fp32 residual stream needs no clamp
    d = (torch.randn(T, H, device=dev())).to(torch.bfloat16)
    db = torch.randn(H, device=dev())
    w = torch.rand(H, device=dev()) + 0.5
    for opw in (False, True):
        xa, xb = x.clone(), x.clone()
        got = K().rmsnorm(xa, w, 1e-5, delta=d, dbias=db, one_plus_w=opw)
        want = ref.rmsnorm(xb, w, 1e-5, delta=d, dbias=db, one_plus_w=opw)
        assert torch.allclose(xa, xb, atol=1e-5) and torch.isfinite(got.float()).all()
        assert rel_err(got, want) < 5e-3
    got = K().rmsnorm(x.clone(), w, 1e-5)
    assert rel_err(got, ref.rmsnorm(x.clone(), w, 1e-5)) < 5e-3


def test_glu_and_gates():
    x = torch.randn(33, 2 * 48, device=dev()).to(torch.bfloat16) * 4
    for act in (ref.ACT_SWIGLU, ref.ACT_SWIGLU_OAI, ref.ACT_GEGLU):
        assert rel_err(K().glu(x, act), ref.glu(x, act)) < 1e-2
    a = torch.randn(100, 64, device=dev()).to(torch.bfloat16)
    g = torch.randn(100, 64, device=dev()).to(torch.bfloat16)
    assert rel_err(K().sigmoid_mul(a, g), ref.sigmoid_mul(a, g)) < 1e-2
    o1 = torch.randn(100, 64, device=dev())
    o2 = o1.clone()
    gl = torch.randn(100, device=dev())
    K().scaled_add(o1, a, gl)
    ref.scaled_add(o2, a, gl)
    assert torch.allclose(o1, o2, atol=1e-4)
    xx = torch.randn(50, 128, device=dev())
    z = torch.randn(50, 128, device=dev()).to(torch.bfloat16)
    w = torch.rand(128, device=dev())
    assert rel_err(K().gated_rmsnorm(xx, z, w, 1e-6), ref.gated_rmsnorm(xx, z, w, 1e-6)) < 1e-2


def _rope_tables(max_pos, n_rot, theta=10000.0):
    inv = theta ** (-torch.arange(0, n_rot, 2, dtype=torch.float32) / n_rot)
    ang = torch.arange(max_pos, dtype=torch.float32)[:, None] * inv[None]
    return torch.cos(ang).to(dev()), torch.sin(ang).to(dev())


@pytest.mark.parametrize("cfg", [dict(n_q=4, n_kv=2, hd=64, n_rot=64, gate=False, norm=False, bias=True),
                                 dict(n_q=8, n_kv=2, hd=128, n_rot=128, gate=False, norm=True, bias=False),
                                 dict(n_q=4, n_kv=1, hd=256, n_rot=64, gate=True, norm=True, bias=False),
                                 dict(n_q=4, n_kv=1, hd=512, n_rot=512, gate=False, norm=True, bias=False, v_norm=True)])
@pytest.mark.parametrize("T", [19, 100])          # 100 rows: the token-major (prefill) form of the kernel
def test_qkv_post(cfg, T):
    bs, nblk = 128, 4
    n_q, n_kv, hd = cfg["n_q"], cfg["n_kv"], cfg["hd"]
    cols = n_q * hd * (2 if cfg["gate"] else 1) + 2 * n_kv * hd
    qkv = torch.randn(T, cols, device=dev()).to(torch.bfloat16)
    bias = torch.randn(cols, device=dev()) if cfg["bias"] else None
    qn = torch.rand(hd, device=dev()) if cfg["norm"] else None
    kn = torch.rand(hd, device=dev()) if cfg["norm"] else None
    pos = torch.arange(100, 100 + T, dtype=torch.int32, device=dev())
    cos, sin = _rope_tables(256, cfg["n_rot"])
    slots = (torch.arange(T, device=dev()) + 130).to(torch.int64)
    slots[3] = -1
    kc = [torch.zeros(nblk, n_kv, bs, hd, dtype=torch.bfloat16, device=dev()) for _ in range(2)]
    vc = [torch.zeros_like(kc[0]) for _ in range(2)]
    extra = {"v_norm": True} if cfg.get("v_norm") else {}       # Gemma-4: weightless RMS norm on V, head_dim 512
    q1, g1 = K().qkv_post(qkv, bias, qn, kn, pos, cos, sin, slots, kc[0], vc[0], n_q, n_kv, hd, cfg["n_rot"], q_gate=cfg["gate"], **extra)
    q2, g2 = ref.qkv_post(qkv, bias, qn, kn, pos, cos, sin, slots, kc[1], vc[1], n_q, n_kv, hd, cfg["n_rot"], q_gate=cfg["gate"], **extra)
    assert rel_err(q1, q2) < 1e-2 and rel_err(kc[0], kc[1]) < 1e-2 and rel_err(vc[0], vc[1]) < 1e-2
    if cfg["gate"]:
        assert rel_err(g1, g2) < 1e-2


def _paged_case(B, q_lens, kv_lens, n_q, n_kv, hd, bs=128, seed=0):
    torch.manual_seed(seed)
    max_blocks = max((L + bs - 1) // bs for L in kv_lens)
    nblk = B * max_blocks + 1
    kc = torch.randn(nblk, n_kv, bs, hd, device=dev()).to(torch.bfloat16)
    vc = torch.randn(nblk, n_kv, bs, hd, device=dev()).to(torch.bfloat16)
    perm = torch.randperm(nblk - 1)[: B * max_blocks].reshape(B, max_blocks) + 1
    bt = perm.to(torch.int32).to(dev())
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev())
    q = torch.randn(sum(q_lens), n_q, hd, device=dev()).to(torch.bfloat16)
    sl = torch.tensor(kv_lens, dtype=torch.int32, device=dev())
    return q, kc, vc, bt, sl, cu


@pytest.mark.parametrize("hd,n_q,n_kv", [(64, 16, 2), (128, 8, 2), (256, 4, 1), (512, 4, 2)])
@pytest.mark.parametrize("window", [0, 128])
def test_attention_decode_and_prefill(hd, n_q, n_kv, window):
    sinks = torch.randn(n_q, device=dev())
    # decode: 3 sequences, one query each, different context lengths; forced split counts
    q, kc, vc, bt, sl, cu = _paged_case(3, [1, 1, 1], [1, 300, 515], n_q, n_kv, hd)
    for splits in (1, 3, None):
        got = K().attention(q, kc, vc, bt, sl, cu, 1, sinks=sinks, window=window, n_splits=splits)
        want = ref.attention(q, kc, vc, bt, sl, cu, 1, sinks=sinks, window=window)
        assert rel_err(got, want) < 1e-2, splits
    # prefill / verify: ragged query lengths, causal, continuing an existing context
    q, kc, vc, bt, sl, cu = _paged_case(3, [70, 5, 130], [70, 205, 400], n_q, n_kv, hd, seed=1)
    got = K().attention(q, kc, vc, bt, sl, cu, 130, window=window, softcap=30.0)
    want = ref.attention(q, kc, vc, bt, sl, cu, 130, window=window, softcap=30.0)
    assert rel_err(got, want) < 1e-2
    # algebraic identity: constant V rows -> output equals that constant when there is no sink
    vc.fill_(0.25)
    got = K().attention(q, kc, vc, bt, sl, cu, 130, window=window)
    assert torch.allclose(got.float(), torch.full_like(got.float(), 0.25), atol=2e-3)


def _quantise_cache(c):
    """bf16 pages -> (int8 pages, per-row fp32 scales) with the cache's own rule: scale = max|x| / 127."""
    f = c.float()
    amax = f.abs().amax(-1)
    sc = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    return torch.round(f / sc.unsqueeze(-1)).clamp(-127, 127).to(torch.int8), sc


@pytest.mark.parametrize("T", [37, 90])
def test_qkv_post_int8_cache_rows(T):
    bs, nblk, n_q, n_kv, hd = 128, 3, 8, 2, 128
    cols = n_q * hd + 2 * n_kv * hd
    qkv = (torch.randn(T, cols, device=dev()) * 3).to(torch.bfloat16)
    kn = torch.rand(hd, device=dev())
    pos = torch.arange(50, 50 + T, dtype=torch.int32, device=dev())
    cos, sin = _rope_tables(256, hd)
    slots = (torch.arange(T, device=dev()) + 120).to(torch.int64)
    slots[5] = -1
    got = [torch.zeros(nblk, n_kv, bs, hd, dtype=torch.int8, device=dev()) for _ in range(2)]
    gs = [torch.ones(nblk, n_kv, bs, device=dev()) for _ in range(2)]
    want = [torch.zeros(nblk, n_kv, bs, hd, dtype=torch.bfloat16, device=dev()) for _ in range(2)]
    q1, _ = K().qkv_post(qkv, None, kn, kn, pos, cos, sin, slots, got[0], got[1], n_q, n_kv, hd, hd, kv_scales=(gs[0], gs[1]))
    q2, _ = ref.qkv_post(qkv, None, kn, kn, pos, cos, sin, slots, want[0], want[1], n_q, n_kv, hd, hd)
    assert rel_err(q1, q2) < 1e-2
    for g8, sc, w in zip(got, gs, want):
        deq = g8.float() * sc.unsqueeze(-1)
        # every element within one quantisation step (plus the oracle's own bf16 rounding) of the unquantised row
        assert bool(((deq - w.float()).abs() <= sc.unsqueeze(-1) * 0.51 + w.float().abs() * 0.005 + 1e-6).all())
        wmax = w.float().abs().amax(-1)
        written = wmax > 0
        assert torch.allclose(sc[written], wmax[written] / 127.0, rtol=1e-2)
        assert bool((sc[~written] == 1).all()) and bool((g8[~written] == 0).all())     # untouched rows (incl. the skipped token)


@pytest.mark.parametrize("hd,n_q,n_kv", [(64, 16, 2), (128, 8, 2), (256, 4, 1)])
@pytest.mark.parametrize("window", [0, 128])
def test_attention_int8_cache(hd, n_q, n_kv, window):
    sinks = torch.randn(n_q, device=dev())
    # decode over int8 pages, several split counts
    q, kc, vc, bt, sl, cu = _paged_case(3, [1, 1, 1], [1, 300, 515], n_q, n_kv, hd)
    (k8, ks), (v8, vs) = _quantise_cache(kc), _quantise_cache(vc)
    want = ref.attention(q, k8, v8, bt, sl, cu, 1, sinks=sinks, window=window, kv_scales=(ks, vs))
    assert rel_err(want, ref.attention(q, kc, vc, bt, sl, cu, 1, sinks=sinks, window=window)) < 3e-2      # the format itself is close to bf16
    for splits in (1, 3, None):
        got = K().attention(q, k8, v8, bt, sl, cu, 1, sinks=sinks, window=window, n_splits=splits, kv_scales=(ks, vs))
        assert rel_err(got, want) < 1e-2, splits
    # prefill: CUDA-core kernel (soft-cap) and, for head dims it supports, page expansion + the tensor-core kernel
    q, kc, vc, bt, sl, cu = _paged_case(3, [70, 5, 130], [70, 205, 400], n_q, n_kv, hd, seed=1)
    (k8, ks), (v8, vs) = _quantise_cache(kc), _quantise_cache(vc)
    got = K().attention(q, k8, v8, bt, sl, cu, 130, window=window, softcap=30.0, kv_scales=(ks, vs))
    assert rel_err(got, ref.attention(q, k8, v8, bt, sl, cu, 130, window=window, softcap=30.0, kv_scales=(ks, vs))) < 1e-2
    want = ref.attention(q, k8, v8, bt, sl, cu, 130, sinks=sinks, window=window, kv_scales=(ks, vs))
    for max_kv in (0, 400):
        got = K().attention(q, k8, v8, bt, sl, cu, 130, sinks=sinks, window=window, kv_scales=(ks, vs), max_kv_len=max_kv)
        K().check_status()
        assert rel_err(got, want) < 1.5e-2, max_kv


@pytest.mark.parametrize("hd,n_q,n_kv", [(64, 16, 2), (128, 8, 2), (256, 4, 2)])
@pytest.mark.parametrize("window", [0, 128])
@pytest.mark.parametrize("use_sinks,softcap", [(False, 0.0), (True, 0.0), (False, 30.0)])
def test_attention_prefill_tensor_core(hd, n_q, n_kv, window, use_sinks, softcap):
    # tcgen05 FlashAttention against the oracle: ragged batch, fresh prompts and continued contexts,
    # tiles on the diagonal, at the window edge and at the sequence end
    sinks = torch.randn(n_q, device=dev()) if use_sinks else None
    q, kc, vc, bt, sl, cu = _paged_case(4, [300, 64, 129, 128], [300, 700, 129, 1024], n_q, n_kv, hd, seed=2)
    got = K().attention_prefill_tc(q, kc, vc, bt, sl, cu, 300, sinks=sinks, window=window, softcap=softcap)
    K().check_status()
    want = ref.attention(q, kc, vc, bt, sl, cu, 300, sinks=sinks, window=window, softcap=softcap)
    assert rel_err(got, want) < 1.5e-2
    # the dispatcher sends long query segments to the same kernel
    assert torch.equal(K().attention(q, kc, vc, bt, sl, cu, 300, sinks=sinks, window=window, softcap=softcap), got)


@pytest.mark.parametrize("hd", [64, 128, 256])
def test_attention_prefill_rescales_its_accumulator_when_the_maximum_grows(hd):
    # keys whose scores grow along the sequence: the running maximum rises by far more than 2^8 between tiles, so the output
    # accumulator in TMEM has to be rescaled in place several times; and a flat case in which it never is
    n_q, n_kv = 4, 2
    for growth in (0.0, 0.06):
        q, kc, vc, bt, sl, cu = _paged_case(2, [700, 256], [700, 1024], n_q, n_kv, hd, seed=7)
        ramp = 1.0 + growth * torch.arange(128, device=dev(), dtype=torch.float32).view(1, 1, 128, 1)
        page_rank = torch.zeros(kc.shape[0], device=dev())
        for b in range(bt.shape[0]):
            page_rank[bt[b].long()] = torch.arange(bt.shape[1], device=dev(), dtype=torch.float32)
        kc = (kc.float() * (ramp + growth * 128 * page_rank.view(-1, 1, 1, 1))).to(torch.bfloat16)
        q = (q.float().abs() * 2).to(torch.bfloat16)
        got = K().attention_prefill_tc(q, kc, vc, bt, sl, cu, 700)
        K().check_status()
        want = ref.attention(q, kc, vc, bt, sl, cu, 700)
        assert rel_err(got, want) < 2e-2, growth


def test_sampling():
    V = 5003
    logits = torch.randn(4, V, device=dev())
    logits[0, 10] = logits[0, 4000] = 50.0       # tie -> lowest id
    assert K().argmax(logits).tolist() == ref.argmax(logits).tolist() and int(K().argmax(logits)[0]) == 10
    # wide vocabulary: split reduction, ties across chunk borders still go to the lowest id, repeated calls reuse the scratch
    wide = torch.randn(3, 201088, device=dev())
    wide[1, 200000] = wide[1, 777] = 60.0
    wide[2, 201087] = 70.0
    for _ in range(3):
        got = K().argmax(wide).tolist()
        assert got == ref.argmax(wide).tolist() and got[1] == 777 and got[2] == 201087
    ids = torch.full((4, 6), -1, dtype=torch.int32, device=dev())
    ids[0, :3] = torch.tensor([10, 77, 4000])
    ids[2, :2] = torch.tensor([5, 6])
    pen = torch.tensor([1.3, 1.0, 2.0, 1.1], device=dev())
    a, b = logits.clone(), logits.clone()
    K().rep_penalty(a, ids, pen)
    ref.rep_penalty(b, ids, pen)
    assert torch.allclose(a, b)
    temp = torch.tensor([0.0, 0.8, 1.0, 1.5], device=dev())
    top_k = torch.tensor([0, 40, 5, 0], dtype=torch.int32, device=dev())
    top_p = torch.tensor([1.0, 0.9, 1.0, 0.5], device=dev())
    min_p = torch.tensor([0.0, 0.0, 0.05, 0.0], device=dev())
    rng1 = torch.tensor([1, 88172645463325252, 1234567, 99], dtype=torch.int64, device=dev())
    rng2 = rng1.clone().cpu()
    for _ in range(5):
        got = K().sample(logits, temp, top_k, top_p, min_p, rng1)
        want = ref.sample(logits.cpu(), temp.cpu(), top_k.cpu(), top_p.cpu(), min_p.cpu(), rng2)
        assert got.cpu().tolist() == want.tolist()
    assert rng1.cpu().tolist() == rng2.tolist()


def test_run_twice_is_bit_identical():
    qw = make_weight(WFormat.MXFP4, 512, 1024)
    x = torch.randn(300, 1024, device=dev()).to(torch.bfloat16)
    a, b = K().gemm(x, qw, out_f32=True), K().gemm(x, qw, out_f32=True)
    assert torch.equal(a, b)
