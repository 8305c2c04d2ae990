"""Launchers for the sm_100a kernels (``csrc/cuda``): torch tensors in, raw pointers out via ctypes.

Every function has a twin with the same signature in :mod:`ops.ref`.  Nothing here falls back
to PyTorch math: a missing or failing kernel raises.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _lib
from .ref import ACT_GEGLU, ACT_NONE, ACT_SWIGLU, ACT_SWIGLU_OAI, MOE_TILE, MoePacking, moe_max_rows
from .weights import QuantWeight, WFormat

_vp = C.c_void_p


class KernelError(RuntimeError):
    pass


def _p(t: Optional[torch.Tensor]):
    return _vp(0) if t is None else _vp(t.data_ptr())


def _stream():
    return _vp(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str):
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


def _planes(w: QuantWeight):
    return int(w.fmt), _p(w.p0), _p(w.p1), _p(w.p2), _p(w.p3)


_launch_count = 0


def launches() -> int:
    """Number of kernel-launching calls made through this module (bench bookkeeping)."""
    return _launch_count


def _count(n=1):
    global _launch_count
    _launch_count += n


def check_status():
    """Synchronise and raise if any kernel recorded a bounded-wait timeout or bad argument."""
    v = _lib.cuda().mx_status_read_and_clear()
    if v:
        names = {1: "TMA producer wait", 2: "MMA wait", 3: "epilogue wait", 4: "dequant producer wait", 5: "peer flag wait",
                 6: "bad argument", 7: "softmax wait"}
        raise KernelError(f"kernel status {v}: {names.get(v, 'unknown')} ran out of its time limit")


def set_gemv_path(path) -> None:
    """Which decode GEMV kernel runs: "auto" (per case, the default), "register" (register-streamed kernels only) or
    "stream" (the bulk-copy streaming kernel wherever it applies); booleans mean register / auto."""
    code = {"auto": 0, "register": 1, "stream": 2, True: 1, False: 0}[path]
    _lib.cuda().mx_gemv_set_path(code)


def set_gemv_bf16_wide(on: bool) -> None:
    """Streaming GEMV over bf16 weights with eight consumer warps per CTA instead of four (MX_GEMV_BF16_WIDE=0/1 sets it at import)."""
    _lib.cuda().mx_gemv_stream_set_bf16_wide(int(bool(on)))


def set_gemv_tma(on: bool) -> None:
    """Streaming GEMV with chunked rows (K above one chunk): one tiled TMA load per plane and stage (default) or one bulk copy per row."""
    _lib.cuda().mx_gemv_stream_set_tma(int(bool(on)))


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the decode-chain kernels (default on): the next kernel's CTAs are scheduled while
    the previous kernel drains and the streaming GEMV prefetches its weights before its inputs exist."""
    _lib.cuda().mx_set_pdl(1 if on else 0)


_sm_count = 0


def sm_count() -> int:
    """Streaming multiprocessors of the current device (148 on a B200), asked once."""
    global _sm_count
    if not _sm_count:
        _sm_count = int(_lib.cuda().mx_sm_count())
    return _sm_count


def _profiled(name):
    """The ops that only exist on the GPU report to the per-op profiler themselves (the CPU/GPU dispatcher wraps the others)."""
    def deco(fn):
        import functools
        from ..utils.profiler import profiler as _prof

        @functools.wraps(fn)
        def wrapped(*args, **kwargs):
            if _prof.enabled:
                return _prof.record(name, fn, args, kwargs)
            return fn(*args, **kwargs)
        return wrapped
    return deco


# ------------------------------------------------------------------ elementwise
def embed(w: QuantWeight, ids, scale: float = 1.0):
    T = ids.numel()
    out = torch.empty(T, w.K, dtype=torch.float32, device=ids.device)
    fmt, p0, p1, p2, p3 = _planes(w)
    _check(_lib.cuda().mx_embed(fmt, p0, p1, p2, p3, _p(ids), _p(out), T, w.K, w.N, C.c_float(scale), _stream()), "embed")
    _count()
    return out


def rmsnorm(x, w, eps, delta=None, dbias=None, one_plus_w=False, delta_scale=1.0, write_x=True, want_out=True):
    T, H = x.shape
    out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device) if want_out else None
    is_f32 = 1 if (delta is not None and delta.dtype == torch.float32) else 0
    if delta is not None:
        assert delta.is_contiguous() and delta.shape == x.shape
    _check(_lib.cuda().mx_rmsnorm(_p(x), _p(delta), is_f32, _p(dbias), _p(w), _p(out), C.c_float(eps), T, H, int(one_plus_w),
                                  C.c_float(delta_scale), int(write_x), _stream()), "rmsnorm")
    _count()
    return out


class CombineDelta:
    """The weighted sum of expert outputs that has not been formed: ``y`` [rows, H] bf16, the packed position of every (token, slot)
    pair (negative = not on this rank) and the routing weights [T, K].  ``rmsnorm_combine`` folds it into the residual inside the
    next norm; ``materialize`` forms it."""

    def __init__(self, y, pair_to_packed, w):
        self.y, self.pair_to_packed, self.w = y, pair_to_packed, w
        self.shape = (w.shape[0], y.shape[1])

    def materialize(self):
        return moe_combine(self.y, MoePacking(None, None, None, self.pair_to_packed, None, None, self.y.shape[0], self.w.shape[1]), self.w)

    def index_select(self, dim, rows):
        assert dim == 0
        return self.materialize().index_select(0, rows)


@_profiled("rmsnorm_combine")
def rmsnorm_combine(x, w, eps, d: "CombineDelta", one_plus_w=False, delta_scale=1.0, want_out=True):
    T, H = x.shape
    out = torch.empty(T, H, dtype=torch.bfloat16, device=x.device) if want_out else None
    _check(_lib.cuda().mx_rmsnorm_combine(_p(x), _p(d.y), _p(d.pair_to_packed), _p(d.w), d.w.shape[1], _p(w), _p(out), C.c_float(eps), T, H,
                                          int(one_plus_w), C.c_float(delta_scale), _stream()), "rmsnorm_combine")
    _count()
    return out


def glu(x, act, alpha=1.702, limit=7.0):
    T, F2 = x.shape
    out = torch.empty(T, F2 // 2, dtype=torch.bfloat16, device=x.device)
    _check(_lib.cuda().mx_glu(_p(x), _p(out), C.c_longlong(T), F2 // 2, act, C.c_float(alpha), C.c_float(limit), _stream()), "glu")
    _count()
    return out


def sigmoid_mul(x, g):
    y = torch.empty_like(x)
    _check(_lib.cuda().mx_sigmoid_mul(_p(x), _p(g), _p(y), C.c_longlong(x.numel()), _stream()), "sigmoid_mul")
    _count()
    return y


def scaled_add(out, src, gate_logit=None):
    _check(_lib.cuda().mx_scaled_add(_p(out), _p(src), _p(gate_logit), out.shape[-1], C.c_longlong(out.numel()), _stream()), "scaled_add")
    _count()
    return out


def gated_rmsnorm(x, z, w, eps):
    rows, hd = x.shape
    y = torch.empty(rows, hd, dtype=torch.bfloat16, device=x.device)
    _check(_lib.cuda().mx_gated_rmsnorm(_p(x), _p(z), _p(w), _p(y), rows, hd, C.c_float(eps), _stream()), "gated_rmsnorm")
    _count()
    return y


def gated_rmsnorm_heads(x, z, w, eps, hd):
    T = x.shape[0]
    n_h = x.shape[1] // hd
    assert x.dtype == torch.float32 and x.is_contiguous() and z.dtype == torch.bfloat16 and z.stride(1) == 1
    y = torch.empty(T, n_h * hd, dtype=torch.bfloat16, device=x.device)
    _check(_lib.cuda().mx_gated_rmsnorm_ld(_p(x), _p(z), z.stride(0), _p(w), _p(y), T, n_h, hd, C.c_float(eps), _stream()), "gated_rmsnorm")
    _count()
    return y


def conv1d_silu(x, w, state, state_slots, cu_q, max_q_len, ckpt=None):
    T, Cc = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and w.dtype == torch.float32 and w.is_contiguous() and state.dtype == torch.bfloat16
    y = torch.empty(T, Cc, dtype=torch.bfloat16, device=x.device)
    _check(_lib.cuda().mx_conv1d_silu(_p(x), x.stride(0), Cc, w.shape[1], _p(w), _p(state), _p(state_slots), _p(cu_q), cu_q.numel() - 1, T,
                                      int(max_q_len), _p(y), _p(ckpt), _stream()), "conv1d_silu")
    _count(1 if max_q_len == 1 else 2)
    return y


DELTANET_CHUNKED_MIN_T = 128      # batches of at least this many tokens take the chunked tensor-core scan (no checkpoints there)


def deltanet_scan(qkv, n_k, ab, a_idx, b_idx, k_of_v, ssm_a, dt_bias, state, state_slots, cu_q, n_v, eps=1e-6, ckpt=None, chunked=None):
    """``chunked``: None picks the chunked (WY) tensor-core kernel for prefill-sized batches without checkpoints and the sequential
    kernel otherwise; True / False force one (tests, benches)."""
    T = qkv.shape[0]
    D = 128
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and ab.dtype == torch.bfloat16 and ab.stride(1) == 1 and state.dtype == torch.float32
    out = torch.empty(T, n_v * D, dtype=torch.float32, device=qkv.device)
    if chunked is None:
        chunked = ckpt is None and T >= DELTANET_CHUNKED_MIN_T
    if chunked:
        assert ckpt is None, "the chunked scan keeps no per-position checkpoints"
        B = cu_q.numel() - 1
        lib = _lib.cuda()
        lib.mx_deltanet_chunk_ws_bytes.restype = C.c_longlong
        ws = torch.empty(int(lib.mx_deltanet_chunk_ws_bytes(T, B, n_v)), dtype=torch.uint8, device=qkv.device)
        egl = torch.empty((T // 64 + B) * n_v, dtype=torch.float32, device=qkv.device)
        _check(lib.mx_deltanet_scan_chunked(_p(qkv), qkv.stride(0), 0, n_k * D, 2 * n_k * D, _p(ab), ab.stride(0), _p(a_idx), _p(b_idx), _p(k_of_v),
                                            _p(ssm_a), _p(dt_bias), _p(state), _p(state_slots), _p(cu_q), B, T, n_v, D,
                                            C.c_float(1.0 / math.sqrt(D)), C.c_float(eps), _p(out), _p(ws), _p(egl), _stream()), "deltanet_scan_chunked")
        _count(2)
        return out
    _check(_lib.cuda().mx_deltanet_scan(_p(qkv), qkv.stride(0), 0, n_k * D, 2 * n_k * D, _p(ab), ab.stride(0), _p(a_idx), _p(b_idx), _p(k_of_v),
                                        _p(ssm_a), _p(dt_bias), _p(state), _p(state_slots), _p(cu_q), cu_q.numel() - 1, n_v, D,
                                        C.c_float(1.0 / math.sqrt(D)), C.c_float(eps), _p(out), _p(ckpt), _stream()), "deltanet_scan")
    _count()
    return out


def qkv_post(qkv, bias, q_norm_w, k_norm_w, positions, rope_cos, rope_sin, slot_map, k_cache, v_cache, n_q, n_kv, hd, n_rot,
             q_gate=False, norm_one_plus_w=False, eps=1e-6, kv_scales=None, v_norm=False):
    T = qkv.shape[0]
    q = torch.empty(T, n_q, hd, dtype=torch.bfloat16, device=qkv.device)
    gate = torch.empty(T, n_q, hd, dtype=torch.bfloat16, device=qkv.device) if q_gate else None
    bs = k_cache.shape[2]
    max_pos = rope_cos.shape[0] if rope_cos is not None else 1
    if kv_scales is not None:
        assert k_cache.dtype == torch.int8 and kv_scales[0].dtype == torch.float32
    else:
        assert k_cache.dtype == torch.bfloat16
    ks, vs = kv_scales if kv_scales is not None else (None, None)
    _check(_lib.cuda().mx_qkv_post_kv8(_p(qkv), _p(bias), _p(q_norm_w), _p(k_norm_w), _p(positions), _p(rope_cos), _p(rope_sin),
                                       _p(slot_map), _p(q), _p(gate), _p(k_cache), _p(v_cache), _p(ks), _p(vs), T, n_q, n_kv, hd, n_rot, bs,
                                       int(q_gate) | (2 if v_norm else 0), int(norm_one_plus_w), C.c_float(eps), max_pos, _stream()), "qkv_post")
    _count()
    return q, gate


# ------------------------------------------------------------------ linear layers
GEMV_MAX_M = 8


def _pick_bn(M: int, N: int) -> int:
    # small-M problems are weight-read bound: use narrow tiles so every SM streams weights
    sms = sm_count()
    if M <= 128:
        for bn in (128, 64, 32):
            if (N + bn - 1) // bn >= sms:
                return bn
        return 32
    tiles128 = ((M + 127) // 128) * ((N + 127) // 128)
    return 128 if tiles128 >= sms else 64


def _gemm_a(x, w: QuantWeight):
    """Activations in the dtype the tensor-core path of this weight format multiplies in."""
    want = torch.bfloat16
    return x if x.dtype == want else x.to(want)


import os as _os

# dense quantised GEMMs with at least this many rows decode the weight once to bf16 first (MX_DEQUANT_ONCE_MIN_M overrides).  Measured on
# Llama-3-8B Q4_K_M, ms per prefill step without -> with: 64 rows 12.3 -> 11.6, 256 rows 16.5 -> 12.8, 512 rows 27.5 -> 17.2,
# 2048 rows 89.6 -> 46.2; batches of 9..63 rows were not measured and keep the in-kernel decode
DEQUANT_ONCE_MIN_M = int(_os.environ.get("MX_DEQUANT_ONCE_MIN_M", "64"))
if _os.environ.get("MX_GEMV_BF16_WIDE") is not None:
    set_gemv_bf16_wide(_os.environ["MX_GEMV_BF16_WIDE"] not in ("", "0"))


def _out_kind(dtype) -> int:
    return {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}[dtype]


def linear(x, w: QuantWeight, bias=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, out_f32=False, row_scale=None, out=None):
    """``out``: write into this [M, n_out] view (unit column stride; a column slice of a wider matrix is fine), so that projections
    whose weights differ in format can share one output without a concatenation."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[-1] == w.K and w.E == 1
    M = x.shape[0]
    if w.fmt == WFormat.EXL3:
        assert act == ACT_NONE and row_scale is None, "EXL3 layers have no fused activation or row scale"
        return _exl3_linear(x, w, bias, out_f32, out)
    n_out = w.N // 2 if act != ACT_NONE else w.N
    odt = torch.float32 if out_f32 else torch.bfloat16
    if out is None:
        out = torch.empty(M, n_out, dtype=odt, device=x.device)
    assert out.shape == (M, n_out) and out.dtype == odt and (M == 0 or out.stride(1) == 1)
    if M == 0:
        return out
    fmt, p0, p1, p2, p3 = _planes(w)
    lib = _lib.cuda()
    if M <= GEMV_MAX_M and row_scale is None:
        # the GEMV kernels write dense rows: a strided view of more than one row goes through a dense buffer
        dst = out if (M == 1 or out.stride(0) == n_out) else torch.empty(M, n_out, dtype=odt, device=x.device)
        _check(lib.mx_gemv(fmt, p0, p1, p2, p3, _p(x), _p(dst), _p(bias), M, w.N, w.K, int(out_f32), act, C.c_float(act_alpha),
                           C.c_float(act_limit), _vp(0), _vp(0), M, 1, _stream()), "gemv")
        if dst is not out:
            out.copy_(dst)
    else:
        xa = _gemm_a(x, w)
        if M >= DEQUANT_ONCE_MIN_M and fmt != int(WFormat.BF16):
            # long chunk, quantised dense weight: decode it once to bf16 and multiply with the TMA-fed kernel (the in-kernel decode
            # repeats per 128-row activation tile).  The scratch matrix is an ordinary allocation: stream-ordered, graph-safe.
            wb = torch.empty(w.N, w.K, dtype=torch.bfloat16, device=x.device)
            _check(lib.mx_dequant_bf16(fmt, p0, p1, p2, p3, C.c_longlong(w.N), w.K, _p(wb), _stream()), "dequant_bf16")
            _count()
            fmt, p0, p1, p2, p3 = int(WFormat.BF16), _p(wb), _vp(0), _vp(0), _vp(0)
        _check(lib.mx_gemm(_p(xa), fmt, p0, p1, p2, p3, 1, _p(out), out.stride(0), int(out_f32), _p(bias), _p(row_scale), act,
                           C.c_float(act_alpha), C.c_float(act_limit), M, w.N, w.K, _vp(0), _vp(0), _pick_bn(M, w.N), _stream()), "gemm")
    _count()
    return out


EXL3_GEMV_MAX_M = 8


def hadamard128(x, pre=None, post=None, bias=None, out_f32=False, out=None):
    """Normalised 128-point Sylvester Hadamard transform of every aligned run of 128 elements of the rows of ``x`` (bf16 or fp32, unit
    column stride): ``had128(x * pre) * post + bias`` with optional fp32 vectors.  ``out``: a [rows, n] view with unit column stride.
    A 3-D fp32 ``x`` [parts, rows, n] (contiguous) stands for the sum of its parts (the partial sums of a K-split product)."""
    nsum, sum_stride = 1, 0
    if x.dim() == 3:
        assert x.dtype == torch.float32 and x.is_contiguous()
        nsum, sum_stride = x.shape[0], x.shape[1] * x.shape[2]
        x = x[0]
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype in (torch.bfloat16, torch.float32) and x.shape[1] % 128 == 0
    rows, n = x.shape
    odt = torch.float32 if out_f32 else torch.bfloat16
    if out is None:
        out = torch.empty(rows, n, dtype=odt, device=x.device)
    assert out.shape == (rows, n) and out.dtype == odt and (rows == 0 or out.stride(1) == 1)
    for v in (pre, post, bias):
        assert v is None or (v.dtype == torch.float32 and v.numel() == n and v.is_contiguous())
    if rows:
        _check(_lib.cuda().mx_hadamard128_cuda(_p(x), int(x.dtype == torch.float32), _p(pre), _p(post), _p(bias), _p(out), int(out_f32),
                                               C.c_longlong(rows), n, x.stride(0), out.stride(0), nsum, C.c_longlong(sum_stride), _stream()), "hadamard128")
        _count()
    return out


def exl3_dequant(w: QuantWeight) -> torch.Tensor:
    """The rotated weight W_rot of an EXL3 layer as bf16 [N, K] (without the Hadamard transforms and the sign / scale vectors)."""
    assert w.fmt == WFormat.EXL3
    wb = torch.empty(w.N, w.K, dtype=torch.bfloat16, device=w.device)
    _check(_lib.cuda().mx_exl3_dequant_bf16(_p(w.p0), w.K // 16, w.N // 16, w.bits, _p(wb), _stream()), "exl3 dequant")
    _count()
    return wb


def _exl3_linear(x, w: QuantWeight, bias, out_f32, out):
    """y = had128(had128(x * suh) W_rot) * svh + bias: the trellis is decoded in registers for decode-sized batches and once to a bf16
    scratch matrix for the tensor-core GEMM otherwise (src/ops/gemv_exl3.cpp:162 runs the same three steps)."""
    M = x.shape[0]
    lib = _lib.cuda()
    xh = hadamard128(x, pre=w.p1[0])
    if M == 0:
        return hadamard128(torch.empty(0, w.N, dtype=torch.float32, device=x.device), out_f32=out_f32, out=out)
    if M <= EXL3_GEMV_MAX_M:
        # the K tiles are cut into ranges (more CTAs for narrow matrices); the partial sums meet in the Hadamard kernel below
        ranges = lib.mx_exl3_gemv_ranges(w.K // 16, w.N // 16)
        acc = torch.empty(ranges, M, w.N, dtype=torch.float32, device=x.device)
        _check(lib.mx_exl3_gemv(_p(w.p0), w.K // 16, w.N // 16, w.bits, _p(xh), _p(acc), M, ranges, _stream()), "exl3 gemv")
        _count()
    else:
        wb = exl3_dequant(w)
        acc = torch.empty(M, w.N, dtype=torch.float32, device=x.device)
        _check(lib.mx_gemm(_p(xh), int(WFormat.BF16), _p(wb), _vp(0), _vp(0), _vp(0), 1, _p(acc), w.N, 1, _vp(0), _vp(0), ACT_NONE, C.c_float(0.0),
                           C.c_float(0.0), M, w.N, w.K, _vp(0), _vp(0), _pick_bn(M, w.N), _stream()), "gemm")
        _count()
    return hadamard128(acc, post=w.p2[0], bias=bias, out_f32=out_f32, out=out)


def gemm(x, w: QuantWeight, bias=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, out_f32=False, row_scale=None, bn=None):
    """Always the tcgen05 path (tests and benches)."""
    M = x.shape[0]
    n_out = w.N // 2 if act != ACT_NONE else w.N
    out = torch.empty(M, n_out, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    fmt, p0, p1, p2, p3 = _planes(w)
    xa = _gemm_a(x, w)
    _check(_lib.cuda().mx_gemm(_p(xa), fmt, p0, p1, p2, p3, 1, _p(out), n_out, int(out_f32), _p(bias), _p(row_scale), act,
                               C.c_float(act_alpha), C.c_float(act_limit), M, w.N, w.K, _vp(0), _vp(0), bn or _pick_bn(M, w.N), _stream()), "gemm")
    _count()
    return out


def grouped_linear(xp, w: QuantWeight, tile_expert, num_tiles, bias=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, out_f32=False, bn=128,
                   out_dtype=None):
    """``out_dtype`` (bf16 / fp16 / fp32) overrides ``out_f32``; fp16 feeds a following MXFP4 GEMM without a cast."""
    P = xp.shape[0]
    n_out = w.N // 2 if act != ACT_NONE else w.N
    odt = out_dtype or (torch.float32 if out_f32 else torch.bfloat16)
    out = torch.empty(P, n_out, dtype=odt, device=xp.device)
    fmt, p0, p1, p2, p3 = _planes(w)
    xp = _gemm_a(xp, w)
    _check(_lib.cuda().mx_gemm(_p(xp), fmt, p0, p1, p2, p3, w.E, _p(out), n_out, _out_kind(odt), _p(bias), _vp(0), act, C.c_float(act_alpha),
                               C.c_float(act_limit), P, w.N, w.K, _p(tile_expert), _p(num_tiles), bn, _stream()), "grouped gemm")
    _count()
    return out


def expert_gemv(x, w: QuantWeight, slot_expert, x_div=1, bias=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, slot_scale=None, out_f32=False,
                e_lo=0):
    """``w`` holds experts [e_lo, e_lo + w.E); slots routed to other experts produce zero rows (expert parallelism)."""
    S = slot_expert.numel()
    n_out = w.N // 2 if act != ACT_NONE else w.N
    out = torch.empty(S, n_out, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    fmt, p0, p1, p2, p3 = _planes(w)
    _check(_lib.cuda().mx_gemv_experts(fmt, p0, p1, p2, p3, _p(x), _p(out), _p(bias), w.N, w.K, int(out_f32), act, C.c_float(act_alpha),
                                       C.c_float(act_limit), _p(slot_expert), _p(slot_scale), S, x_div, int(e_lo), int(e_lo) + w.E, _stream()),
           "expert gemv")
    _count()
    return out


# ------------------------------------------------------------------ attention
_attn_scratch: dict = {}


TC_PREFILL_MIN_Q = 64      # query segments at least this long take the tensor-core kernel


def attention_prefill_tc(q, k_cache, v_cache, block_table, seq_lens, cu_q, max_q_len, sinks=None, window=0, scale=None, softcap=0.0):
    """tcgen05 FlashAttention (head_dim 64 / 128 / 256, page size 128, optional logit soft-cap)."""
    Tq, n_q, hd = q.shape
    n_kv, bs = k_cache.shape[1], k_cache.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    out = torch.empty(Tq, n_q, hd, dtype=torch.bfloat16, device=q.device)
    _check(_lib.cuda().mx_attention_prefill_tc(_p(q), _p(k_cache), _p(v_cache), _p(block_table), _p(seq_lens), _p(cu_q), _p(sinks), _p(out),
                                               seq_lens.numel(), Tq, int(max_q_len), n_q, n_kv, hd, block_table.shape[1], k_cache.shape[0], bs,
                                               int(window), C.c_float(scale), C.c_float(softcap or 0.0), _stream()), "attention_prefill_tc")
    _count()
    return out


_kv8_scratch: dict = {}


def _dequant_pages(k_cache, v_cache, kv_scales, block_table, seq_lens, max_kv_len):
    """The pages of this batch of an int8 cache as a bf16 scratch cache [B * nb, n_kv, bs, hd] with its own block table."""
    _, n_kv, bs, hd = k_cache.shape
    B = seq_lens.numel()
    nb = block_table.shape[1] if max_kv_len <= 0 else min(block_table.shape[1], (max_kv_len + bs - 1) // bs)
    need = 2 * B * nb * n_kv * bs * hd
    buf = _kv8_scratch.get(k_cache.device)
    if buf is None or buf.numel() < need:
        buf = torch.zeros(need, dtype=torch.bfloat16, device=k_cache.device)      # zeros: pages that are never filled stay finite
        _kv8_scratch[k_cache.device] = buf
    dk = buf[: need // 2].view(B * nb, n_kv, bs, hd)
    dv = buf[need // 2: need].view(B * nb, n_kv, bs, hd)
    key = (k_cache.device, "table", B, nb)
    table = _kv8_scratch.get(key)
    if table is None:
        table = torch.arange(B * nb, dtype=torch.int32, device=k_cache.device).view(B, nb)
        _kv8_scratch[key] = table
    _check(_lib.cuda().mx_kv_dequant_pages(_p(k_cache), _p(v_cache), _p(kv_scales[0]), _p(kv_scales[1]), _p(block_table), _p(seq_lens),
                                           _p(dk), _p(dv), B, n_kv, bs, hd, block_table.shape[1], nb, _stream()), "kv_dequant_pages")
    _count()
    return dk, dv, table


ATTN_MAX_SPLITS = 32


def attention(q, k_cache, v_cache, block_table, seq_lens, cu_q, max_q_len, sinks=None, window=0, scale=None, softcap=0.0, n_splits=None,
              kv_scales=None, max_kv_len=0):
    Tq, n_q, hd = q.shape
    n_kv, bs = k_cache.shape[1], k_cache.shape[2]
    B = seq_lens.numel()
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    assert (k_cache.dtype == torch.int8) == (kv_scales is not None)
    if max_q_len >= TC_PREFILL_MIN_Q and hd in (64, 128, 256) and bs == 128 and n_splits is None:
        if kv_scales is not None:       # the tensor-core kernel reads bf16 pages: expand this batch's pages first
            dk, dv, table = _dequant_pages(k_cache, v_cache, kv_scales, block_table, seq_lens, max_kv_len)
            return attention_prefill_tc(q, dk, dv, table, seq_lens, cu_q, max_q_len, sinks=sinks, window=window, scale=scale, softcap=softcap)
        return attention_prefill_tc(q, k_cache, v_cache, block_table, seq_lens, cu_q, max_q_len, sinks=sinks, window=window, scale=scale,
                                    softcap=softcap)
    if n_splits is None:
        # decode-sized problems: split the KV range so that ~2 CTAs per SM exist
        ctas = B * n_kv * max(1, (max_q_len * (n_q // n_kv) + 31) // 32)
        max_kv_tiles = max(1, (block_table.shape[1] * bs) // 64)
        # (the cap: with two KV heads of 256 and one sequence, 128 ranges instead of 32 took a 16k context from 119 to 103 us but a 4k
        # context from 48 to 54 us -- the last CTA's merge grows with the ranges; the kernel itself takes any number)
        n_splits = max(1, min(max_kv_tiles, ATTN_MAX_SPLITS, (2 * sm_count()) // max(ctas, 1)))
    need = n_splits * Tq * n_q * (hd + 2)
    if torch.cuda.is_current_stream_capturing():
        # a captured kernel keeps the raw address: the scratch must live exactly as long as the graph, so it comes from the
        # graph's own pool.  (The shared buffer below is re-allocated when a larger request arrives; a graph that had
        # captured its old address would then write through a dangling pointer.)
        buf = torch.empty(need, dtype=torch.float32, device=q.device)
    else:
        buf = _attn_scratch.get(q.device)
        if buf is None or buf.numel() < need:
            buf = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q.device)
            _attn_scratch[q.device] = buf
    o_part = buf[: n_splits * Tq * n_q * hd]
    ml_part = buf[n_splits * Tq * n_q * hd: need]
    out = torch.empty(Tq, n_q, hd, dtype=torch.bfloat16, device=q.device)
    if kv_scales is not None:
        _check(_lib.cuda().mx_attention_kv8(_p(q), _p(k_cache), _p(v_cache), _p(kv_scales[0]), _p(kv_scales[1]), _p(block_table), _p(seq_lens),
                                            _p(cu_q), _p(sinks), _p(out), _p(o_part), _p(ml_part), B, Tq, int(max_q_len), n_q, n_kv, hd,
                                            block_table.shape[1], bs, int(window), C.c_float(scale), C.c_float(softcap), int(n_splits),
                                            _stream()), "attention_kv8")
    else:
        _check(_lib.cuda().mx_attention(_p(q), _p(k_cache), _p(v_cache), _p(block_table), _p(seq_lens), _p(cu_q), _p(sinks), _p(out),
                                        _p(o_part), _p(ml_part), B, Tq, int(max_q_len), n_q, n_kv, hd, block_table.shape[1], bs, int(window),
                                        C.c_float(scale), C.c_float(softcap), int(n_splits), _stream()), "attention")
    _count(_lib.cuda().mx_attention_launches(B, int(max_q_len), n_q, n_kv))
    return out


# ------------------------------------------------------------------ MoE
def moe_route(logits, bias, k, renorm=True):
    T, E = logits.shape
    idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    _check(_lib.cuda().mx_moe_route(_p(logits), _p(bias), T, E, k, int(renorm), _p(idx), _p(w), _stream()), "moe_route")
    _count()
    return idx, w


def moe_pack(topk_idx, E, e_lo=0, e_hi=None, tile=MOE_TILE):
    e_hi = E if e_hi is None else e_hi
    T, K = topk_idx.shape
    dev = topk_idx.device
    n = T * K
    max_rows = moe_max_rows(n, e_hi - e_lo) if tile > 1 else max(n, 1)
    counts = torch.empty(E, dtype=torch.int32, device=dev)
    seg = torch.empty(E + 1, dtype=torch.int32, device=dev)
    packed_token = torch.empty(max_rows, dtype=torch.int32, device=dev)
    pair_to_packed = torch.empty(n, dtype=torch.int32, device=dev)
    tile_expert = torch.zeros(max(max_rows // MOE_TILE, 1), dtype=torch.int32, device=dev)
    tile_valid = torch.zeros(max(max_rows // MOE_TILE, 1), dtype=torch.int32, device=dev) if tile > 1 else None
    num_tiles = torch.empty(2, dtype=torch.int32, device=dev)
    _check(_lib.cuda().mx_moe_pack(_p(topk_idx), n, K, E, e_lo, e_hi, _p(counts), _p(seg), _p(packed_token), _p(pair_to_packed),
                                   _p(tile_expert), _p(num_tiles), max_rows, int(tile), _p(tile_valid), _stream()), "moe_pack")
    _count()
    return MoePacking(counts, seg, packed_token, pair_to_packed, tile_expert, num_tiles, max_rows, K, tile_valid)


@_profiled("moe_quant")
def moe_quant(x, rows, max_tiles, rows_per_tile, src_index=None, x_div=1, row_limit=None):
    """bf16 rows -> MXFP8 rows + scale atoms for :func:`mxf4_gemm` (see ``mx_moe_quant``).  Returns (xq [rows, KB*128] uint8,
    sfx [KB, max_tiles, 512] uint8).  Rows that are skipped (negative index, beyond ``row_limit``) are left unwritten."""
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    K = x.shape[1]
    KB = (K + 127) // 128
    xq = torch.empty(rows, KB * 128, dtype=torch.uint8, device=x.device)
    sfx = torch.empty(KB, max_tiles, 512, dtype=torch.uint8, device=x.device)
    _check(_lib.cuda().mx_moe_quant(_p(x), x.stride(0), _p(src_index), int(x_div), _p(row_limit), int(rows), K, int(max_tiles),
                                    int(rows_per_tile), _p(xq), _p(sfx), _stream()), "moe_quant")
    _count()
    return xq, sfx


@_profiled("moe_route_quant")
def moe_route_quant(logits, bias, k, x, renorm=True, w_copies=1):
    """Decode: router top-k and pair-mode MXFP8 quantisation of the T rows of ``x`` in one launch.  Returns (idx, w, xq, sfx); ``w`` is
    [T, w_copies * k], the k weights repeated (one per partial row when the down projection splits K)."""
    T, E = logits.shape
    Kd = x.shape[1]
    KB = (Kd + 127) // 128
    n = T * k
    idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, w_copies * k, dtype=torch.float32, device=logits.device)
    xq = torch.empty(n, KB * 128, dtype=torch.uint8, device=x.device)
    sfx = torch.empty(KB, n, 512, dtype=torch.uint8, device=x.device)
    _check(_lib.cuda().mx_moe_route_quant(_p(logits), _p(bias), T, E, k, int(renorm), _p(idx), _p(w), int(w_copies), _p(x), x.stride(0), Kd, n, _p(xq), _p(sfx),
                                          _stream()), "moe_route_quant")
    _count()
    return idx, w, xq, sfx


GEMV_NORM_MAX_M = 2      # the fused prologue normalises its rows one after the other; more rows take the separate kernel


@_profiled("gemv_norm")
def gemv_norm(x, norm_w, eps, w: QuantWeight, bias=None, delta=None, one_plus_w=False, delta_scale=1.0, out_f32=False, want_h=False, route=None):
    """Decode (at most GEMV_NORM_MAX_M rows of at most 4096 elements): residual add + RMSNorm + dense GEMV in one launch (``csrc/cuda/gemv_stream.cu``).  ``x`` fp32 [T, H] is
    not modified; ``delta`` is None, a bf16 [T, H] tensor or a :class:`CombineDelta`.  Returns None when the shape or the weight format
    is not taken, else ``(y, x_new, h)``: the product, the updated residual (``x`` itself without a delta) and, with ``want_h``, the
    normalised rows.  ``route = (router_bias, k, renorm, w_copies)`` makes ``w`` the router: the last CTA also picks the top-k experts
    and writes the rows as MXFP8 pair tiles, and the result is ``(logits, x_new, h, idx, topk_w, xq, sfx)`` with ``topk_w`` of shape
    [T, w_copies * k] (the k weights repeated: one per partial row when the down projection splits K)."""
    T, H = x.shape
    if T > GEMV_NORM_MAX_M or H > 4096 or w.E != 1 or w.fmt not in (WFormat.BF16, WFormat.Q8) or x.dtype != torch.float32 or not x.is_contiguous():
        return None
    comb = delta if isinstance(delta, CombineDelta) else None
    if delta is not None and comb is None and not (isinstance(delta, torch.Tensor) and delta.dtype == torch.bfloat16 and delta.is_contiguous()):
        return None
    if comb is not None and comb.w.shape[1] > 8:
        return None
    dev = x.device
    fmt, p0, p1, _, _ = _planes(w)
    y = torch.empty(T, w.N, dtype=torch.float32 if (out_f32 or route is not None) else torch.bfloat16, device=dev)
    x_new = torch.empty_like(x) if delta is not None else x
    h = torch.empty(T, H, dtype=torch.bfloat16, device=dev) if want_h else None
    idx = tw = xq = sfx = None
    rb, k, renorm, n, copies = None, 0, 1, 0, 1
    if route is not None:
        rb, k, renorm, copies = route
        KB = (H + 127) // 128
        n = T * k
        idx = torch.empty(T, k, dtype=torch.int32, device=dev)
        tw = torch.empty(T, copies * k, dtype=torch.float32, device=dev)
        xq = torch.empty(n, KB * 128, dtype=torch.uint8, device=dev)
        sfx = torch.empty(KB, n, 512, dtype=torch.uint8, device=dev)
    rc = _lib.cuda().mx_gemv_norm(fmt, p0, p1, _p(x), _p(x_new) if delta is not None else _vp(0), _p(delta) if (delta is not None and comb is None) else _vp(0),
                                  _p(comb.y) if comb is not None else _vp(0), _p(comb.pair_to_packed) if comb is not None else _vp(0),
                                  _p(comb.w) if comb is not None else _vp(0), comb.w.shape[1] if comb is not None else 0, _p(norm_w), C.c_float(eps),
                                  int(one_plus_w), C.c_float(delta_scale), _p(h), _p(y), _p(bias), T, w.N, w.K, int(y.dtype == torch.float32),
                                  int(route is not None), _p(rb), k, int(bool(renorm)), _p(idx), _p(tw), copies, _p(xq), _p(sfx), n, _stream())
    if rc == 1:
        return None
    _check(rc, "gemv_norm")
    _count()
    if route is not None:
        return y, x_new, h, idx, tw, xq, sfx
    return y, x_new, h


def mxf4_ksplit(K: int, want: int) -> int:
    """K ranges ``mxf4_gemm(..., ksplit=want)`` really uses for a reduction length K: every range owns at least one 128-element block."""
    kb = (K + 127) // 128
    per = (kb + max(want, 1) - 1) // max(want, 1)
    return (kb + per - 1) // per


@_profiled("mxf4_gemm")
def mxf4_gemm(w: QuantWeight, xq, sfx, tile_expert, max_tiles, row_stride, tile_valid=None, default_valid=128, num_tiles=None, e_lo=0,
              bias0=None, bias1=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, zero_out=False, ksplit=1):
    """Block-scaled MXFP4 x MXFP8 grouped GEMM on the tensor cores (``csrc/cuda/gemm_mxf4.cu``).  ``w`` is an MXF4T bank and
    ``xq``/``sfx`` come from :func:`moe_quant` or from a gated call of this function.  A plain bank returns bf16 [rows, N]; a gated
    pair (``w.dual``, with ``act``) returns the activation already quantised for the next projection: (oq [rows, N rounded up to
    128] uint8, osf scale atoms).  Rows that belong to no live tile are left unwritten unless ``zero_out``.  ``ksplit`` > 1 (plain banks):
    K is cut into that many ranges and the result has ``ksplit`` x rows rows, range s in rows [s * rows, (s + 1) * rows): partial sums
    that the consumer adds (decode, where a handful of pairs would otherwise leave most SMs idle)."""
    assert w.fmt == WFormat.MXF4T
    rows = xq.shape[0]
    dev = xq.device
    out = oq = osf = None
    oq_ld = 0
    if w.dual:
        oq_ld = (w.N + 127) // 128 * 128
        oq = torch.empty(rows, oq_ld, dtype=torch.uint8, device=dev)
        osf = torch.empty(oq_ld // 128, max_tiles, 512, dtype=torch.uint8, device=dev)
    else:
        ksplit = mxf4_ksplit(w.K, ksplit)
        out = (torch.zeros if zero_out else torch.empty)(ksplit * rows, w.N, dtype=torch.bfloat16, device=dev)
    _check(_lib.cuda().mx_mxf4_gemm(_p(w.p0), _p(w.p1), int(w.dual), w.E, _p(xq), _p(sfx), rows, w.N, w.K, _p(tile_expert), _p(tile_valid),
                                    int(default_valid), _p(num_tiles), int(max_tiles), int(row_stride), int(e_lo), _p(bias0), _p(bias1),
                                    _p(out), w.N, _p(oq), _p(osf), oq_ld, int(act), C.c_float(act_alpha), C.c_float(act_limit), int(ksplit), _stream()),
           "mxf4 gemm")
    _count()
    return (oq, osf) if w.dual else out


def expert_group_gemv(x, w: QuantWeight, pk: MoePacking, x_index=None, bias=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, e_lo=0):
    """Batched-decode MoE GEMV over a compact packing (``moe_pack(..., tile=1)``): every local expert streams its weights once
    and multiplies them with all rows routed to it (8 rows per pass).  Row r of the output belongs to packed position r;
    its input is ``x[x_index[r]]`` (gate|up reads the token rows in place) or ``x[r]`` (down)."""
    P = pk.max_rows
    n_out = w.N // 2 if act != ACT_NONE else w.N
    out = torch.empty(P, n_out, dtype=torch.bfloat16, device=x.device)
    fmt, p0, p1, p2, p3 = _planes(w)
    _check(_lib.cuda().mx_gemv_group(fmt, p0, p1, p2, p3, _p(x), _p(x_index), _p(out), _p(bias), w.N, w.K, act, C.c_float(act_alpha),
                                     C.c_float(act_limit), _p(pk.counts), _p(pk.seg_start), int(e_lo), w.E, _stream()), "gemv_group")
    _count()
    return out


def moe_gather(x, pk: MoePacking, f16=False, zero_pad=False):
    """Rows of ``x`` in packed order.  Padding rows of the expert tiles are left unwritten unless ``zero_pad`` (no consumer reads them:
    a grouped GEMM row depends on its own input row only)."""
    H = x.shape[1]
    xp = torch.empty(pk.max_rows, H, dtype=torch.float16 if f16 else torch.bfloat16, device=x.device)
    _check(_lib.cuda().mx_moe_gather(_p(x), _p(pk.packed_token), _p(pk.num_tiles), _p(xp), H, pk.max_rows, int(f16), int(zero_pad), _stream()), "moe_gather")
    _count()
    return xp


def moe_combine(yp, pk: MoePacking, w, out=None, accumulate=False):
    assert yp.dtype == torch.bfloat16
    T, K = w.shape
    H = yp.shape[1]
    if out is None:
        out = torch.empty(T, H, dtype=torch.float32, device=yp.device)
        accumulate = False
    _check(_lib.cuda().mx_moe_combine(_p(yp), _p(pk.pair_to_packed), _p(w), _p(out), int(out.dtype == torch.float32), T, H, K,
                                      int(accumulate), _stream()), "moe_combine")
    _count()
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits):
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(_lib.cuda().mx_argmax(_p(logits), rows, V, logits.stride(0), _p(out), _stream()), "argmax")
    _count()
    return out


def rep_penalty(logits, ids, penalty):
    rows, V = logits.shape
    _check(_lib.cuda().mx_rep_penalty(_p(logits), rows, V, logits.stride(0), _p(ids), ids.shape[1], _p(penalty), _stream()), "rep_penalty")
    _count()
    return logits


def sample(logits, temperature, top_k, top_p, min_p, rng):
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _check(_lib.cuda().mx_sample(_p(logits), rows, V, logits.stride(0), _p(temperature), _p(top_k), _p(top_p), _p(min_p), _p(rng), _p(out),
                                 _stream()), "sample")
    _count()
    return out
