"""The block-scaled MXFP4 x MXFP8 grouped GEMM (csrc/cuda/gemm_mxf4.cu) and its activation quantiser against fp32 PyTorch.

The oracle multiplies the decoded weights with activations rounded by ``ref.mxfp8_roundtrip`` (the same rounding rule as the
kernel), so the comparison isolates the kernel's data movement and accumulation; a second, looser check against the
unrounded activations bounds what the 8-bit activations cost.
"""
import pytest
import torch

from machx_inference_engine_b200.ops import ref
from machx_inference_engine_b200.ops.weights import WFormat, from_dense, to_mxf4_tiles

pytestmark = pytest.mark.gpu


def K():
    from machx_inference_engine_b200.ops import cuda
    return cuda


def dev():
    return torch.device("cuda:0")


def rel_err(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def bank(N, Kd, E, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    w = from_dense(torch.randn(E, N, Kd, generator=g) * 0.05, WFormat.MXFP4).to(dev())
    return w, to_mxf4_tiles(w)


def decode_quant(xq, sfb, rows, Kd, rows_per_tile):
    """(xq, sfb) of moe_quant -> fp32 [rows, Kd]."""
    KB = sfb.shape[0]
    r = torch.arange(rows, device=xq.device)
    tile, rin = r // rows_per_tile, r % rows_per_tile
    idx = ((rin % 32) * 16 + (rin // 32) * 4)[:, None] + torch.arange(4, device=xq.device)[None, :]      # [rows, 4] bytes in the atom
    ex = torch.stack([sfb[kb][tile].long().gather(1, idx) for kb in range(KB)], dim=1)                 # [rows, KB, 4]
    scale = torch.exp2(ex.reshape(rows, KB * 4).float() - 127.0)
    vals = xq[:rows].view(torch.float8_e4m3fn).float().reshape(rows, KB * 4, 32) * scale.unsqueeze(-1)
    return vals.reshape(rows, KB * 128)[:, :Kd]


@pytest.mark.parametrize("Kd", [2880, 256])
def test_activation_quantiser_matches_the_oracle_rounding(Kd):
    torch.manual_seed(0)
    rows = 200
    x = (torch.randn(rows, Kd, device=dev()) * torch.rand(rows, 1, device=dev()) * 8).to(torch.bfloat16)
    x[3] = 0
    x[5, :40] *= 1000.0
    xq, sfb = K().moe_quant(x, rows, 2, 128)
    torch.cuda.synchronize()
    got = decode_quant(xq, sfb, rows, Kd, 128)
    want = ref.mxfp8_roundtrip(x)
    assert torch.equal(got, want), rel_err(got, want)
    # the columns between K and the padded width are zeros
    if xq.shape[1] > Kd:
        assert int(xq[:, Kd:].view(torch.int8).abs().max()) == 0
    # what 8-bit activations cost on their own
    assert rel_err(want, x) < 4e-2


def _oracle(x_rows, W, e, bias):
    y = ref.mxfp8_roundtrip(x_rows) @ W[e].t()
    return y if bias is None else y + bias[e]


@pytest.mark.parametrize("N,Kd", [(300, 2880), (128, 128), (2880, 512)])
def test_grouped_gemm_packed_segments(N, Kd):
    torch.manual_seed(1)
    E, topk, T = 6, 2, 330
    w, wt = bank(N, Kd, E, 3)
    W = w.dequantize()
    x = torch.randn(T, Kd, device=dev()).to(torch.bfloat16)
    # skewed routing: expert 0 gets many rows (several full tiles), expert 5 none
    logits = torch.randn(T, E, device=dev())
    logits[:, 0] += 2.0
    logits[:, 5] -= 50.0
    idx, _ = K().moe_route(logits, None, topk)
    pk = K().moe_pack(idx, E)
    pk_r = ref.moe_pack(idx, E)
    nt = int(pk.num_tiles[0])
    assert torch.equal(pk.tile_valid[:nt], pk_r.tile_valid[:nt])
    mt = pk.tile_expert.numel()
    xq, sfx = K().moe_quant(x, pk.max_rows, mt, 128, src_index=pk.packed_token, row_limit=pk.num_tiles)
    bias = torch.randn(E, N, device=dev()) * 0.1
    y = K().mxf4_gemm(wt, xq, sfx, pk.tile_expert, mt, 128, tile_valid=pk.tile_valid, num_tiles=pk.num_tiles, bias0=bias)
    K().check_status()
    nrows = int(pk.num_tiles[1])
    tok = pk.packed_token[:nrows]
    live = tok >= 0
    row_e = torch.repeat_interleave(pk.tile_expert[:nt].long(), 128)[:nrows]
    want = torch.zeros(nrows, N, device=dev())
    exact = torch.zeros_like(want)
    for e in range(E):
        m = live & (row_e == e)
        if m.any():
            want[m] = _oracle(x[tok[m].long()], W, e, bias)
            exact[m] = x[tok[m].long()].float() @ W[e].t() + bias[e]
    assert rel_err(y[:nrows][live], want[live]) < 4e-3            # bf16 output rounding
    assert rel_err(y[:nrows][live], exact[live]) < 4e-2           # what the 8-bit activations cost


@pytest.mark.parametrize("act,F", [(ref.ACT_SWIGLU, 320), (ref.ACT_SWIGLU_OAI, 2880)])
def test_gated_pair_of_banks_and_the_whole_expert_ffn(act, F):
    torch.manual_seed(2)
    E, topk, T, H = 8, 4, 150, 512
    g, _ = bank(F, H, E, 5)
    u, _ = bank(F, H, E, 6)
    d, dt = bank(H, F, E, 7)
    gut = to_mxf4_tiles(g, u)
    Wg, Wu, Wd = g.dequantize(), u.dequantize(), d.dequantize()
    x = torch.randn(T, H, device=dev()).to(torch.bfloat16)
    idx, w = K().moe_route(torch.randn(T, E, device=dev()), None, topk)
    pk = K().moe_pack(idx, E)
    mt = pk.tile_expert.numel()
    tiles = dict(tile_valid=pk.tile_valid, num_tiles=pk.num_tiles)
    gb, ub, db = (torch.randn(E, n, device=dev()) * 0.1 for n in (F, F, H))
    xq, sfx = K().moe_quant(x, pk.max_rows, mt, 128, src_index=pk.packed_token, row_limit=pk.num_tiles)
    aq, sfa = K().mxf4_gemm(gut, xq, sfx, pk.tile_expert, mt, 128, bias0=gb, bias1=ub, act=act, **tiles)
    y = K().mxf4_gemm(dt, aq, sfa, pk.tile_expert, mt, 128, bias0=db, **tiles)
    out = K().moe_combine(y, pk, w)
    K().check_status()
    # the gated projection's own output, decoded, against the oracle's activation
    nrows = int(pk.num_tiles[1])
    a_got = decode_quant(aq, sfa, nrows, F, 128)
    tok = pk.packed_token[:nrows]
    live = tok >= 0
    nt = int(pk.num_tiles[0])
    row_e = torch.repeat_interleave(pk.tile_expert[:nt].long(), 128)[:nrows]
    a_want = torch.zeros(nrows, F, device=dev())
    for e in range(E):
        m = live & (row_e == e)
        if m.any():
            xr = ref.mxfp8_roundtrip(x[tok[m].long()])
            a_want[m] = ref.mxfp8_roundtrip(ref._act(act, xr @ Wg[e].t() + gb[e], xr @ Wu[e].t() + ub[e], 1.702, 7.0).to(torch.bfloat16))
    assert rel_err(a_got[live], a_want[live]) < 2e-2              # one-step flips of e4m3 where fp32 summation order differs
    if aq.shape[1] > F:
        assert int(aq[:nrows][live][:, F:].view(torch.int8).abs().max()) == 0
    # the whole expert FFN
    want = torch.zeros(T, H, device=dev())
    exact = torch.zeros(T, H, device=dev())
    xf = x.float()
    xr = ref.mxfp8_roundtrip(x)
    for e in range(E):
        sel = (idx == e)
        rows = sel.any(dim=1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        wk = (w * sel)[rows].sum(dim=1, keepdim=True)
        av = ref._act(act, xr[rows] @ Wg[e].t() + gb[e], xr[rows] @ Wu[e].t() + ub[e], 1.702, 7.0).to(torch.bfloat16)
        want[rows] += wk * (ref.mxfp8_roundtrip(av) @ Wd[e].t() + db[e]).to(torch.bfloat16).float()
        ae = ref._act(act, xf[rows] @ Wg[e].t() + gb[e], xf[rows] @ Wu[e].t() + ub[e], 1.702, 7.0)
        exact[rows] += wk * (ae @ Wd[e].t() + db[e])
    assert rel_err(out, want) < 1e-2
    assert rel_err(out, exact) < 5e-2


def test_pair_mode_decode_rows_and_foreign_experts():
    torch.manual_seed(3)
    E, topk, T, H, F = 8, 4, 3, 2880, 256
    g, _ = bank(F, H, E, 8)
    u, _ = bank(F, H, E, 9)
    d, dt = bank(H, F, E, 10)
    gut = to_mxf4_tiles(g, u)
    Wg, Wu, Wd = g.dequantize(), u.dequantize(), d.dequantize()
    x = torch.randn(T, H, device=dev()).to(torch.bfloat16)
    idx, _ = K().moe_route(torch.randn(T, E, device=dev()), None, topk)
    n = T * topk
    te = idx.reshape(-1)
    xq, sfx = K().moe_quant(x, n, n, 1, x_div=topk)
    aq, sfa = K().mxf4_gemm(gut, xq, sfx, te, n, 1, default_valid=1, act=ref.ACT_SWIGLU_OAI)
    y = K().mxf4_gemm(dt, aq, sfa, te, n, 1, default_valid=1)
    K().check_status()
    a_got = decode_quant(aq, sfa, n, F, 1)
    for i in range(n):
        e = int(te[i])
        xr = ref.mxfp8_roundtrip(x[i // topk: i // topk + 1])
        a_want = ref.mxfp8_roundtrip(ref._act(ref.ACT_SWIGLU_OAI, xr @ Wg[e].t(), xr @ Wu[e].t(), 1.702, 7.0).to(torch.bfloat16))
        assert rel_err(a_got[i:i + 1], a_want) < 2e-2, i
        assert rel_err(y[i:i + 1], a_got[i:i + 1] @ Wd[e].t()) < 6e-3, i
    # expert parallelism: the banks hold experts [2, 5); pairs of other experts are skipped and stay zero
    lo, hi = 2, 5
    aq2, sfa2 = K().mxf4_gemm(gut.slice_experts(lo, hi), xq, sfx, te, n, 1, default_valid=1, act=ref.ACT_SWIGLU_OAI, e_lo=lo)
    y2 = K().mxf4_gemm(dt.slice_experts(lo, hi), aq2, sfa2, te, n, 1, default_valid=1, e_lo=lo, zero_out=True)
    K().check_status()
    own = (te >= lo) & (te < hi)
    assert torch.equal(y2[own], y[own]) and int(y2[~own].abs().max() if (~own).any() else 0) == 0


def test_run_twice_is_bit_identical():
    torch.manual_seed(4)
    E, T, H, F = 4, 260, 256, 256
    _, wt = bank(F, H, E, 11)
    x = torch.randn(T, H, device=dev()).to(torch.bfloat16)
    idx, _ = K().moe_route(torch.randn(T, E, device=dev()), None, 2)
    pk = K().moe_pack(idx, E)
    mt = pk.tile_expert.numel()
    outs = []
    for _ in range(2):
        xq, sfx = K().moe_quant(x, pk.max_rows, mt, 128, src_index=pk.packed_token, row_limit=pk.num_tiles)
        y = K().mxf4_gemm(wt, xq, sfx, pk.tile_expert, mt, 128, tile_valid=pk.tile_valid, num_tiles=pk.num_tiles, zero_out=True)
        nrows = int(pk.num_tiles[1])
        live = pk.packed_token[:nrows] >= 0
        outs.append(y[:nrows][live].clone())
    assert torch.equal(outs[0], outs[1])


def test_decode_fusions_match_their_unfused_forms():
    """route + quantise in one launch, and the expert combine folded into the residual add + RMSNorm: bit-identical to the
    separate kernels."""
    torch.manual_seed(9)
    T, H, E, topk = 5, 2880, 32, 4
    x = torch.randn(T, H, device=dev()).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev())
    rb = torch.randn(E, device=dev()) * 0.1
    idx, w = K().moe_route(logits, rb, topk)
    xq, sfx = K().moe_quant(x, T * topk, T * topk, 1, x_div=topk)
    idx2, w2, xq2, sfx2 = K().moe_route_quant(logits, rb, topk, x)
    K().check_status()
    assert torch.equal(idx, idx2) and torch.equal(w, w2) and torch.equal(xq, xq2)
    rows = torch.arange(T * topk, device=dev())
    for kb in range(sfx.shape[0]):
        assert torch.equal(sfx[kb, rows, :4], sfx2[kb, rows, :4])          # row 0 of each pair's atom: bytes 0..3
    # combine inside the norm
    y = torch.randn(T * topk + 3, H, device=dev()).to(torch.bfloat16)
    p2p = torch.arange(T * topk, dtype=torch.int32, device=dev())
    p2p[2] = -1                                                            # a pair that lives on another rank
    res = torch.randn(T, H, device=dev())
    nw = torch.rand(H, device=dev()) + 0.5
    d = K().CombineDelta(y, p2p, w)
    x1, x2 = res.clone(), res.clone()
    out1 = K().rmsnorm(x1, nw, 1e-5, delta=d.materialize(), delta_scale=0.5)
    out2 = K().rmsnorm_combine(x2, nw, 1e-5, d, delta_scale=0.5)
    K().check_status()
    assert torch.equal(x1, x2) and torch.equal(out1, out2)


def test_down_projection_k_split_partials_add_up():
    """ksplit = 2 leaves two partial rows per pair (k-blocks [0, 12) and [12, 23) of K = 2880); their sum is the unsplit product up to
    the bf16 rounding of each partial, and the bias is added once."""
    torch.manual_seed(12)
    E, topk, H, F = 8, 4, 512, 2880
    d, dt = bank(H, F, E, 13)
    bias = torch.randn(E, H, device=dev()) * 0.1
    a = torch.randn(1, F, device=dev()).to(torch.bfloat16)
    te = torch.tensor([5, 1, 6, 2], dtype=torch.int32, device=dev())
    aq, sfa = K().moe_quant(a, topk, topk, 1, x_div=topk)
    y1 = K().mxf4_gemm(dt, aq, sfa, te, topk, 1, default_valid=1, bias0=bias)
    y2 = K().mxf4_gemm(dt, aq, sfa, te, topk, 1, default_valid=1, bias0=bias, ksplit=2)
    K().check_status()
    assert y2.shape == (2 * topk, H)
    assert rel_err(y2[:topk].float() + y2[topk:].float(), y1) < 8e-3
    Wd = d.dequantize()
    aw = decode_quant(aq, sfa, topk, F, 1)
    for i in range(topk):
        e = int(te[i])
        lo = aw[i:i + 1, :12 * 128] @ Wd[e][:, :12 * 128].t() + bias[e]
        hi = aw[i:i + 1, 12 * 128:] @ Wd[e][:, 12 * 128:].t()
        assert rel_err(y2[i:i + 1], lo) < 6e-3 and rel_err(y2[topk + i:topk + i + 1], hi) < 6e-3, i


@pytest.mark.parametrize("T,kind", [(1, "none"), (2, "bf16"), (1, "combine"), (2, "combine")])
def test_norm_fused_into_the_gemv_and_router_tail(T, kind):
    """Residual add + RMSNorm inside the GEMV that consumes it, against the separate kernels; the router form also routes and writes
    the MXFP8 pair tiles in the same launch."""
    torch.manual_seed(20 + T)
    H, N, E, topk = 2880, 640, 32, 4
    res = torch.randn(T, H, device=dev())
    nw = torch.rand(H, device=dev()) + 0.5
    w = from_dense(torch.randn(1, N, H) * 0.02, WFormat.BF16).to(dev())
    bias = torch.randn(N, device=dev()) * 0.1
    delta = None
    if kind == "bf16":
        delta = torch.randn(T, H, device=dev()).to(torch.bfloat16)
    elif kind == "combine":
        y = torch.randn(T * topk + 2, H, device=dev()).to(torch.bfloat16)
        p2p = torch.randperm(T * topk + 2, device=dev())[:T * topk].to(torch.int32)
        p2p[1] = -1
        delta = K().CombineDelta(y, p2p, torch.rand(T, topk, device=dev()))
    assert K().gemv_norm(torch.randn(3, H, device=dev()), nw, 1e-5, w, bias) is None        # more rows: not taken
    # separate kernels
    x1 = res.clone()
    if kind == "combine":
        h1 = K().rmsnorm_combine(x1, nw, 1e-5, delta, delta_scale=0.5)
    else:
        h1 = K().rmsnorm(x1, nw, 1e-5, delta=delta, delta_scale=0.5)
    y1 = K().linear(h1, w, bias=bias)
    # fused
    x0 = res.clone()
    y2, x2, h2 = K().gemv_norm(x0, nw, 1e-5, w, bias, delta=delta, delta_scale=0.5, want_h=True)
    K().check_status()
    assert torch.equal(x0, res)                                  # the input residual is not modified
    assert rel_err(x2, x1) < 1e-6 and rel_err(h2, h1) < 4e-3 and rel_err(y2, y1) < 6e-3
    # router form
    rw = from_dense(torch.randn(1, E, H) * 0.05, WFormat.BF16).to(dev())
    rb = torch.randn(E, device=dev()) * 0.1
    for copies in (1, 2):
        logits, x3, h3, idx, tw, xq, sfx = K().gemv_norm(res.clone(), nw, 1e-5, rw, None, delta=delta, delta_scale=0.5, want_h=True,
                                                         route=(rb, topk, True, copies))
        K().check_status()
        assert torch.equal(h3, h2) and torch.equal(x3, x2)
        idx_w, tw_w = K().moe_route(logits, rb, topk)
        xq_w, sfx_w = K().moe_quant(h3, T * topk, T * topk, 1, x_div=topk)
        assert torch.equal(idx, idx_w) and torch.equal(xq, xq_w)
        assert torch.equal(tw.reshape(T, copies, topk), tw_w.unsqueeze(1).expand(T, copies, topk))
        rows = torch.arange(T * topk, device=dev())
        for kb in range(sfx.shape[0]):
            assert torch.equal(sfx[kb, rows, :4], sfx_w[kb, rows, :4])
        assert rel_err(logits, K().linear(h3, rw, out_f32=True)) < 1e-5
