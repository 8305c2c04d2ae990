"""Plain PyTorch fp32 twins of every kernel in ``csrc/cuda`` (same signatures as ``ops.cuda``).

They are the numerical oracle of the GPU tests and the execution path on machines without a
GPU (CPU plumbing runs, gloo multi-process tests).  Shapes, layouts (paged KV, 16-row gate/up
interleave, packed MoE rows) and rounding points (bf16 activations) mirror the kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .weights import QuantWeight

ACT_NONE, ACT_SWIGLU, ACT_SWIGLU_OAI, ACT_GEGLU = 0, 1, 2, 3
MOE_TILE = 128


# Matmul dtype of this module.  fp32 = the numerical oracle of the tests.  The library-baseline arm of the benchmarks (plain PyTorch
# = cuBLAS GEMMs + NCCL on the same model, no kernel of this engine) switches it to bf16 so that its GEMMs run on the tensor cores.
_MM_DTYPE = torch.float32
_DENSE_BUDGET = [None]          # bytes of decoded weights that may stay resident (None = unlimited); what does not fit is decoded per call


def set_matmul_dtype(dtype, dense_budget_bytes=None) -> None:
    global _MM_DTYPE
    _MM_DTYPE = dtype
    _DENSE_BUDGET[0] = dense_budget_bytes


def _mm(a: torch.Tensor, b_t: torch.Tensor) -> torch.Tensor:
    """a [M,K] @ b_t [N,K]^T in the module's matmul dtype, fp32 result."""
    if _MM_DTYPE == torch.float32:
        return a.to(torch.float32) @ b_t.to(torch.float32).t()
    return (a.to(_MM_DTYPE) @ b_t.to(_MM_DTYPE).t()).to(torch.float32)


class _LazyBank:
    """Expert bank decoded one expert at a time (and kept while the residency budget lasts)."""

    def __init__(self, w: QuantWeight):
        self.w, self.cache = w, {}

    def __getitem__(self, e):
        if isinstance(e, torch.Tensor):
            return torch.stack([self[int(i)] for i in e.tolist()])
        d = self.cache.get(e)
        if d is None:
            d = self.w.slice_experts(e, e + 1).dequantize(_MM_DTYPE)[0]
            nbytes = d.numel() * d.element_size()
            if _DENSE_BUDGET[0] is None or _DENSE_BUDGET[0] >= nbytes:
                self.cache[e] = d
                if _DENSE_BUDGET[0] is not None:
                    _DENSE_BUDGET[0] -= nbytes
        return d


def _dense(w: QuantWeight):
    if w._dense_cache is None:
        if _DENSE_BUDGET[0] is not None and w.E > 1:
            w._dense_cache = _LazyBank(w)
        else:
            w._dense_cache = w.dequantize(_MM_DTYPE)
            if _DENSE_BUDGET[0] is not None:
                _DENSE_BUDGET[0] -= w._dense_cache.numel() * w._dense_cache.element_size()
    return w._dense_cache


def embed(w: QuantWeight, ids: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    tbl = _dense(w)[0]
    return tbl[ids.long().clamp(0, w.N - 1)].to(torch.float32) * scale


def rmsnorm(x, w, eps, delta=None, dbias=None, one_plus_w=False, delta_scale=1.0, write_x=True, want_out=True):
    if delta is not None:
        d = delta.to(torch.float32)
        if dbias is not None:
            d = d + dbias
        xs = x + d * delta_scale
        if write_x:
            x.copy_(xs)
    else:
        xs = x
    if not want_out:
        return None
    g = (1.0 + w) if one_plus_w else w
    inv = torch.rsqrt(xs.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xs * inv * g).to(torch.bfloat16)


def _act(act, g, u, alpha, limit):
    if act == ACT_SWIGLU:
        return torch.nn.functional.silu(g) * u
    if act == ACT_SWIGLU_OAI:
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
        return g * torch.sigmoid(alpha * g) * (u + 1.0)
    return torch.nn.functional.gelu(g, approximate="tanh") * u


def _deinterleave16(y: torch.Tensor):
    """[..., 2F] with 16-wide interleaved gate|up groups -> (gate [...,F], up [...,F])."""
    F2 = y.shape[-1]
    v = y.reshape(*y.shape[:-1], F2 // 32, 2, 16)
    return v[..., 0, :].reshape(*y.shape[:-1], F2 // 2), v[..., 1, :].reshape(*y.shape[:-1], F2 // 2)


def glu(x, act, alpha=1.702, limit=7.0):
    g, u = _deinterleave16(x.to(torch.float32))
    return _act(act, g, u, alpha, limit).to(torch.bfloat16)


def linear(x, w: QuantWeight, bias=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, out_f32=False, row_scale=None, out=None):
    if out is not None:
        return out.copy_(linear(x, w, bias, act, act_alpha, act_limit, out_f32, row_scale))
    y = _mm(x, _dense(w)[0])
    if bias is not None:
        y = y + bias
    if act != ACT_NONE:
        g, u = _deinterleave16(y)
        y = _act(act, g, u, act_alpha, act_limit)
    if row_scale is not None:
        y = y * row_scale.unsqueeze(-1)
    return y if out_f32 else y.to(torch.bfloat16)


def hadamard128(x, pre=None, post=None, bias=None, out_f32=False, out=None):
    """``had128(x * pre) * post + bias`` over every aligned run of 128 elements of the rows (EXL3 layers; src/ops/hadamard.cpp:36)."""
    from ..formats.exl3 import hadamard128 as _had
    v = x.to(torch.float32)
    if pre is not None:
        v = v * pre
    v = _had(v)
    if post is not None:
        v = v * post
    if bias is not None:
        v = v + bias
    v = v if out_f32 else v.to(torch.bfloat16)
    return v if out is None else out.copy_(v)


def grouped_linear(xp, w: QuantWeight, tile_expert, num_tiles, bias=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, out_f32=False, bn=128,
                   out_dtype=None):
    """xp: packed rows [P,K]; tile t (rows 128t..128t+127) uses expert tile_expert[t] for t < num_tiles[0]."""
    W = _dense(w)
    P = xp.shape[0]
    n_out = w.N // 2 if act != ACT_NONE else w.N
    out = torch.zeros(P, n_out, dtype=torch.float32, device=xp.device)
    nt = int(num_tiles[0])
    te = tile_expert[:nt].tolist()
    for t, e in enumerate(te):
        rows = slice(t * MOE_TILE, min((t + 1) * MOE_TILE, P))
        y = _mm(xp[rows], W[e])
        if bias is not None:
            y = y + bias[e]
        if act != ACT_NONE:
            g, u = _deinterleave16(y)
            y = _act(act, g, u, act_alpha, act_limit)
        out[rows] = y
    return out.to(out_dtype) if out_dtype is not None else (out if out_f32 else out.to(torch.bfloat16))


def expert_gemv(x, w: QuantWeight, slot_expert, x_div=1, bias=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, slot_scale=None, out_f32=False,
                e_lo=0):
    """y[s] = W[slot_expert[s] - e_lo] @ x[s // x_div]; slots whose expert lies outside [e_lo, e_lo + E) give zero rows."""
    W = _dense(w)
    S = slot_expert.numel()
    rows = torch.arange(S, device=x.device) // x_div
    xe = x.to(torch.float32)[rows]
    se = slot_expert.long() - e_lo
    owned = (se >= 0) & (se < w.E)
    se = se.clamp(0, w.E - 1)
    y = torch.einsum("sk,snk->sn", xe.to(_MM_DTYPE), W[se]).to(torch.float32)
    if bias is not None:
        y = y + bias[se]
    if act != ACT_NONE:
        g, u = _deinterleave16(y)
        y = _act(act, g, u, act_alpha, act_limit)
    y = y * owned.unsqueeze(-1)
    if slot_scale is not None:
        y = y * slot_scale.unsqueeze(-1)
    return y if out_f32 else y.to(torch.bfloat16)


def qkv_post(qkv, bias, q_norm_w, k_norm_w, positions, rope_cos, rope_sin, slot_map, k_cache, v_cache, n_q, n_kv, hd, n_rot,
             q_gate=False, norm_one_plus_w=False, eps=1e-6, kv_scales=None, v_norm=False):
    """Returns (q [T,n_q,hd] bf16, gate or None); writes K/V into the paged cache (int8 rows + scales when kv_scales is given)."""
    T = qkv.shape[0]
    x = qkv.to(torch.float32)
    if bias is not None:
        x = x + bias
    q_stride = 2 * hd if q_gate else hd
    qc = n_q * q_stride
    qpart = x[:, :qc].reshape(T, n_q, q_stride)
    gate = None
    if q_gate:
        gate = qpart[..., hd:].to(torch.bfloat16).contiguous()
        qpart = qpart[..., :hd]
    k = x[:, qc:qc + n_kv * hd].reshape(T, n_kv, hd)
    v = x[:, qc + n_kv * hd:].reshape(T, n_kv, hd)

    def norm(t, w):
        if w is None:
            return t
        g = (1.0 + w) if norm_one_plus_w else w
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * g

    qpart, k = norm(qpart, q_norm_w), norm(k, k_norm_w)
    if v_norm:
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    if n_rot > 0:
        half = n_rot // 2
        pos = positions.long().clamp(0, rope_cos.shape[0] - 1)
        c, s = rope_cos[pos].unsqueeze(1), rope_sin[pos].unsqueeze(1)

        def rope(t):
            a, b = t[..., :half], t[..., half:n_rot]
            return torch.cat([a * c - b * s, a * s + b * c, t[..., n_rot:]], dim=-1)

        qpart, k = rope(qpart), rope(k)
    if n_kv == 0:                   # queries only (a draft head that reads another model's cache)
        return qpart.to(torch.bfloat16).contiguous(), gate
    bs = k_cache.shape[2]
    ok = slot_map >= 0
    blk, off = (slot_map[ok] // bs).long(), (slot_map[ok] % bs).long()
    if kv_scales is not None:
        for cache, sc, t in ((k_cache, kv_scales[0], k[ok]), (v_cache, kv_scales[1], v[ok])):
            amax = t.abs().amax(-1)
            scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
            cache[blk, :, off] = torch.round(t * (1.0 / scale).unsqueeze(-1)).clamp(-127, 127).to(torch.int8)
            sc[blk, :, off] = scale
        return qpart.to(torch.bfloat16).contiguous(), gate
    k_cache[blk, :, off] = k[ok].to(k_cache.dtype)
    v_cache[blk, :, off] = v[ok].to(v_cache.dtype)
    return qpart.to(torch.bfloat16).contiguous(), gate


def attention(q, k_cache, v_cache, block_table, seq_lens, cu_q, max_q_len, sinks=None, window=0, scale=None, softcap=0.0, n_splits=1,
              kv_scales=None, max_kv_len=0):
    """q [Tq,n_q,hd]; caches [blocks,n_kv,bs,hd] (bf16, or int8 with kv_scales = (k_scale, v_scale) [blocks,n_kv,bs]); returns bf16 [Tq,n_q,hd]."""
    Tq, n_q, hd = q.shape
    n_kv, bs = k_cache.shape[1], k_cache.shape[2]
    gqa = n_q // n_kv
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    out = torch.zeros(Tq, n_q, hd, dtype=torch.float32, device=q.device)
    cu = cu_q.tolist()
    for b in range(len(cu) - 1):
        q0, q1 = cu[b], cu[b + 1]
        if q1 <= q0:
            continue
        L = int(seq_lens[b])
        nblk = (L + bs - 1) // bs
        blocks = block_table[b, :nblk].long()
        Kp, Vp = k_cache[blocks].to(torch.float32), v_cache[blocks].to(torch.float32)
        if kv_scales is not None:
            Kp, Vp = Kp * kv_scales[0][blocks].unsqueeze(-1), Vp * kv_scales[1][blocks].unsqueeze(-1)
        K = Kp.permute(1, 0, 2, 3).reshape(n_kv, nblk * bs, hd)[:, :L]
        V = Vp.permute(1, 0, 2, 3).reshape(n_kv, nblk * bs, hd)[:, :L]
        qq = q[q0:q1].to(torch.float32) * scale                                 # [t, n_q, hd]
        Kh = K.repeat_interleave(gqa, dim=0)
        Vh = V.repeat_interleave(gqa, dim=0)
        s = torch.einsum("thd,hkd->htk", qq.to(_MM_DTYPE), Kh.to(_MM_DTYPE)).to(torch.float32)
        if softcap and softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        qpos = torch.arange(L - (q1 - q0), L, device=q.device).unsqueeze(-1)
        kpos = torch.arange(L, device=q.device).unsqueeze(0)
        ok = kpos <= qpos
        if window and window > 0:
            ok = ok & (kpos > qpos - window)
        s = s.masked_fill(~ok.unsqueeze(0), float("-inf"))
        if sinks is not None:
            sk = sinks.to(torch.float32).reshape(n_q, 1, 1).expand(n_q, q1 - q0, 1)
            p = torch.softmax(torch.cat([s, sk], dim=-1), dim=-1)[..., :-1]
        else:
            p = torch.softmax(s, dim=-1)
        out[q0:q1] = torch.einsum("htk,hkd->thd", p.to(_MM_DTYPE), Vh.to(_MM_DTYPE)).to(torch.float32)
    return out.to(torch.bfloat16)


def sigmoid_mul(x, g):
    return (x.to(torch.float32) * torch.sigmoid(g.to(torch.float32))).to(torch.bfloat16)


def scaled_add(out, src, gate_logit=None):
    s = src.to(torch.float32)
    if gate_logit is not None:
        s = s * torch.sigmoid(gate_logit).unsqueeze(-1)
    out.add_(s)
    return out


def gated_rmsnorm(x, z, w, eps):
    """x fp32 [rows,hd], z bf16 [rows,hd]."""
    zz = z.to(torch.float32)
    return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w * torch.nn.functional.silu(zz)).to(torch.bfloat16)


def gated_rmsnorm_heads(x, z, w, eps, hd):
    """x fp32 [T, n_h*hd]; z bf16 [T, n_h*hd] (any row stride); per-head y = w * x/rms(x) * silu(z) -> bf16 [T, n_h*hd]."""
    T = x.shape[0]
    xx = x.reshape(T, -1, hd)
    zz = z.to(torch.float32).reshape(T, -1, hd)
    y = xx * torch.rsqrt(xx.pow(2).mean(-1, keepdim=True) + eps) * w * torch.nn.functional.silu(zz)
    return y.reshape(T, -1).to(torch.bfloat16)


# ------------------------------------------------------------------ gated DeltaNet
def conv1d_silu(x, w, state, state_slots, cu_q, max_q_len, ckpt=None):
    """Depthwise causal conv + SiLU over packed variable-length sequences.

    x bf16 [T, C] (any row stride); w fp32 [C, Kc], tap j multiplies input t-(Kc-1)+j; state bf16 [slots, Kc-1, C]
    holds the Kc-1 inputs before each sequence's next token and is advanced in place; ckpt (optional, bf16
    [T, Kc-1, C]) receives the state as it stands after every position."""
    T, C = x.shape
    Kc = w.shape[1]
    y = torch.empty(T, C, dtype=torch.bfloat16, device=x.device)
    cu = cu_q.tolist()
    for b in range(len(cu) - 1):
        t0, t1 = cu[b], cu[b + 1]
        if t1 <= t0:
            continue
        slot = int(state_slots[b])
        full = torch.cat([state[slot].to(torch.float32), x[t0:t1].to(torch.float32)], dim=0)      # [Kc-1+n, C]
        win = full.unfold(0, Kc, 1)                                                               # [n, C, Kc]
        acc = (win * w.unsqueeze(0)).sum(-1)
        y[t0:t1] = torch.nn.functional.silu(acc).to(torch.bfloat16)
        if ckpt is not None:
            for i in range(t1 - t0):
                ckpt[t0 + i] = full[i + 1:i + Kc].to(torch.bfloat16)
        state[slot] = full[-(Kc - 1):].to(torch.bfloat16)
    return y


def deltanet_scan(qkv, n_k, ab, a_idx, b_idx, k_of_v, ssm_a, dt_bias, state, state_slots, cu_q, n_v, eps=1e-6, ckpt=None):
    """Gated delta rule over packed sequences.

    qkv bf16 [T, (2 n_k + n_v) * 128] = conv output (q heads | k heads | v heads); ab bf16 [T, *] holds the alpha / beta
    logits of v-head h in columns a_idx[h] / b_idx[h]; k_of_v[h] = k-head feeding v-head h.  Per token:
    q, k L2-normalised (q also scaled by 1/sqrt(128)); g = ssm_a * softplus(alpha + dt_bias); beta = sigmoid(.);
    S <- e^g S;  d = (v - S^T k) beta;  S <- S + k d^T;  out = S^T q.   state fp32 [slots, n_v, 128 (v), 128 (k)]
    is advanced in place; ckpt (optional fp32 [T, n_v, 128, 128]) receives S after every position.  Returns fp32 [T, n_v*128]."""
    T, D = qkv.shape[0], 128
    x = qkv.to(torch.float32)
    q = x[:, :n_k * D].reshape(T, n_k, D)
    k = x[:, n_k * D:2 * n_k * D].reshape(T, n_k, D)
    v = x[:, 2 * n_k * D:].reshape(T, n_v, D)
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + eps) / math.sqrt(D)
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + eps)
    kv = k_of_v.long()
    q, k = q[:, kv], k[:, kv]
    abf = ab.to(torch.float32)
    g = ssm_a * torch.nn.functional.softplus(abf[:, a_idx.long()] + dt_bias)
    beta = torch.sigmoid(abf[:, b_idx.long()])
    out = torch.empty(T, n_v, D, dtype=torch.float32, device=qkv.device)
    cu = cu_q.tolist()
    for b in range(len(cu) - 1):
        t0, t1 = cu[b], cu[b + 1]
        if t1 <= t0:
            continue
        slot = int(state_slots[b])
        S = state[slot].clone()
        for t in range(t0, t1):
            S = S * torch.exp(g[t]).reshape(n_v, 1, 1)
            d = (v[t] - torch.einsum("hvk,hk->hv", S, k[t])) * beta[t].unsqueeze(-1)
            S = S + d.unsqueeze(-1) * k[t].unsqueeze(1)
            out[t] = torch.einsum("hvk,hk->hv", S, q[t])
            if ckpt is not None:
                ckpt[t] = S
        state[slot] = S
    return out.reshape(T, n_v * D)


# ------------------------------------------------------------------ MoE
DELTANET_CHUNK = 64


def deltanet_scan_chunked(qkv, n_k, ab, a_idx, b_idx, k_of_v, ssm_a, dt_bias, state, state_slots, cu_q, n_v, eps=1e-6, chunk=DELTANET_CHUNK):
    """The same recurrence as :func:`deltanet_scan` in its chunked (WY) form: the arithmetic of the tensor-core scan kernel, stated
    in fp32.  Within a chunk of C tokens with cumulative log-decay G_i, the per-token corrections U (rows u_i = d_i) solve
        (I + A) U = beta * V - diag(beta e^G) K S0^T,      A_ij = beta_i e^{G_i - G_j} (k_i . k_j) for j < i,
    so with T = (I + A)^-1:  U = T (beta V) - T (beta e^G K) S0^T;  the outputs are O = diag(e^G) Q S0^T + (M * Q K^T) U with
    M_ij = e^{G_i - G_j} for j <= i, and the state leaves the chunk as S = e^{G_last} S0 + U^T diag(e^{G_last - G}) K.
    Sequences are padded to whole chunks with beta = 0, g = 0, k = 0 rows (identity steps).  No per-position checkpoints."""
    T, D = qkv.shape[0], 128
    x = qkv.to(torch.float32)
    q = x[:, :n_k * D].reshape(T, n_k, D)
    k = x[:, n_k * D:2 * n_k * D].reshape(T, n_k, D)
    v = x[:, 2 * n_k * D:].reshape(T, n_v, D)
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + eps) / math.sqrt(D)
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + eps)
    kv = k_of_v.long()
    q, k = q[:, kv], k[:, kv]                                        # [T, n_v, D]
    abf = ab.to(torch.float32)
    g = ssm_a * torch.nn.functional.softplus(abf[:, a_idx.long()] + dt_bias)      # [T, n_v]
    beta = torch.sigmoid(abf[:, b_idx.long()])
    out = torch.empty(T, n_v, D, dtype=torch.float32, device=qkv.device)
    cu = cu_q.tolist()
    C = chunk
    tril = torch.tril(torch.ones(C, C, device=qkv.device), diagonal=-1).bool()
    for b in range(len(cu) - 1):
        t0, t1 = cu[b], cu[b + 1]
        if t1 <= t0:
            continue
        slot = int(state_slots[b])
        S = state[slot].clone()                                      # [n_v, D(v), D(k)]
        for c0 in range(t0, t1, C):
            n = min(C, t1 - c0)
            pad = lambda t: torch.cat([t[c0:c0 + n], t.new_zeros((C - n,) + t.shape[1:])]) if n < C else t[c0:c0 + n]
            qc, kc, vc, gc, bc = (pad(t).transpose(0, 1) for t in (q, k, v, g, beta))      # [n_v, C, ...]
            G = gc.cumsum(-1)                                        # [n_v, C]
            dec = torch.exp(G.unsqueeze(-1) - G.unsqueeze(-2))       # e^{G_i - G_j}
            A = (bc.unsqueeze(-1) * dec * (kc @ kc.transpose(-1, -2))).masked_fill(~tril, 0.0)
            Tm = torch.linalg.solve_triangular(torch.eye(C, device=A.device) + A, torch.eye(C, device=A.device).expand_as(A), upper=False)
            Wv = Tm @ (bc.unsqueeze(-1) * vc)                        # [n_v, C, D(v)]
            Wk = Tm @ ((bc * torch.exp(G)).unsqueeze(-1) * kc)       # [n_v, C, D(k)]
            U = Wv - Wk @ S.transpose(-1, -2)
            Mqk = (dec * (qc @ kc.transpose(-1, -2))).masked_fill(torch.triu(torch.ones(C, C, device=A.device), diagonal=1).bool(), 0.0)
            O = torch.exp(G).unsqueeze(-1) * (qc @ S.transpose(-1, -2)) + Mqk @ U
            Gl = G[:, -1]
            S = torch.exp(Gl).reshape(n_v, 1, 1) * S + U.transpose(-1, -2) @ (torch.exp(Gl.unsqueeze(-1) - G).unsqueeze(-1) * kc)
            out[c0:c0 + n] = O.transpose(0, 1)[:n]
        state[slot] = S
    return out.reshape(T, n_v * D)


def moe_route(logits, bias, k, renorm=True):
    x = logits.to(torch.float32)
    if bias is not None:
        x = x + bias
    # descending value, ties -> lowest index (stable sort on -x)
    order = torch.sort(-x, dim=-1, stable=True).indices[:, :k]
    sel = torch.gather(x, 1, order)
    if renorm:
        w = torch.softmax(sel, dim=-1)
    else:
        w = torch.exp(sel - torch.logsumexp(x, dim=-1, keepdim=True))
    return order.to(torch.int32), w


@dataclass
class MoePacking:
    counts: torch.Tensor          # [E]
    seg_start: torch.Tensor       # [E+1] padded segment starts
    packed_token: torch.Tensor    # [max_rows] token of each packed row (-1 = pad)
    pair_to_packed: torch.Tensor  # [T*K] packed row of each (token, slot) pair, -1 if not owned
    tile_expert: torch.Tensor     # [max_tiles]
    num_tiles: torch.Tensor       # [2]: live tiles, packed rows
    max_rows: int
    K: int
    tile_valid: Optional[torch.Tensor] = None   # [max_tiles] live rows of each tile (block-scaled MXFP4 kernel)


def moe_max_rows(n_pairs: int, n_local_experts: int) -> int:
    return (n_pairs + n_local_experts * (MOE_TILE - 1) + MOE_TILE - 1) // MOE_TILE * MOE_TILE


def moe_pack(topk_idx, E, e_lo=0, e_hi=None, tile=MOE_TILE):
    """``tile`` = 128: segments padded to GEMM tiles; ``tile`` = 1: compact segments (batched-decode GEMV path)."""
    e_hi = E if e_hi is None else e_hi
    T, K = topk_idx.shape
    dev = topk_idx.device
    flat = topk_idx.reshape(-1).long()
    n = flat.numel()
    max_rows = moe_max_rows(n, e_hi - e_lo) if tile > 1 else max(n, 1)
    owned = (flat >= e_lo) & (flat < e_hi)
    counts = torch.bincount(flat[owned], minlength=E)[:E]
    padded = (counts + tile - 1) // tile * tile
    seg = torch.zeros(E + 1, dtype=torch.long, device=dev)
    seg[1:] = torch.cumsum(padded, 0)
    packed_token = torch.full((max_rows,), -1, dtype=torch.int32, device=dev)
    pair_to_packed = torch.full((n,), -1, dtype=torch.int32, device=dev)
    order = torch.sort(torch.where(owned, flat, torch.full_like(flat, E)), stable=True).indices
    n_owned = int(owned.sum())
    order = order[:n_owned]
    e_sorted = flat[order]
    rank_in_e = torch.arange(n_owned, device=dev) - torch.cumsum(counts, 0)[e_sorted] + counts[e_sorted]
    dst = seg[e_sorted] + rank_in_e
    packed_token[dst] = (order // K).to(torch.int32)
    pair_to_packed[order] = dst.to(torch.int32)
    tiles = (padded // MOE_TILE) if tile > 1 else torch.zeros_like(padded)
    tile_expert = torch.repeat_interleave(torch.arange(E, device=dev), tiles).to(torch.int32)
    max_tiles = max(max_rows // MOE_TILE, 1)
    te = torch.zeros(max_tiles, dtype=torch.int32, device=dev)
    te[: tile_expert.numel()] = tile_expert
    num_tiles = torch.tensor([int(tiles.sum()), int(seg[E])], dtype=torch.int32, device=dev)
    tv = torch.zeros(max_tiles, dtype=torch.int32, device=dev)
    if tile > 1 and tile_expert.numel():
        first = torch.repeat_interleave(torch.cumsum(tiles, 0) - tiles, tiles)           # first tile of each tile's expert
        within = torch.arange(tile_expert.numel(), device=dev) - first
        tv[: tile_expert.numel()] = torch.clamp(counts[tile_expert.long()] - within * tile, max=tile).to(torch.int32)
    return MoePacking(counts.to(torch.int32), seg.to(torch.int32), packed_token, pair_to_packed, te, num_tiles, max_rows, K, tv)


def moe_gather(x, pk: MoePacking, f16=False):
    xp = torch.zeros(pk.max_rows, x.shape[1], dtype=torch.float16 if f16 else x.dtype, device=x.device)
    ok = pk.packed_token >= 0
    xp[ok] = x[pk.packed_token[ok].long()].to(xp.dtype)
    return xp


def mxfp8_roundtrip(x: torch.Tensor) -> torch.Tensor:
    """``x`` [..., K] (K a multiple of 32) rounded the way the activation quantiser of the block-scaled MXFP4 kernel rounds it:
    per 32 elements a power-of-two scale, the smallest that keeps the block inside e4m3's range (448), then round-to-nearest
    e4m3.  Returns the decoded fp32 values."""
    xs = x.to(torch.float32).reshape(*x.shape[:-1], x.shape[-1] // 32, 32)
    amax = xs.abs().amax(dim=-1, keepdim=True)
    ex = torch.floor(torch.log2(amax.clamp_min(1e-38))) - 8.0
    ex = torch.where(amax * torch.exp2(-ex) > 448.0, ex + 1.0, ex).clamp_(-126.0, 126.0)
    q = (xs * torch.exp2(-ex)).to(torch.float8_e4m3fn).to(torch.float32)
    return torch.where(amax > 0, q * torch.exp2(ex), torch.zeros_like(q)).reshape(x.shape)


def expert_group_gemv(x, w: QuantWeight, pk: MoePacking, x_index=None, bias=None, act=ACT_NONE, act_alpha=1.702, act_limit=7.0, e_lo=0):
    """y[r] = W[expert of packed row r] @ x[x_index[r] or r] over a compact packing; bf16 [max_rows, N_out]."""
    W = _dense(w)
    P = pk.max_rows
    n_out = w.N // 2 if act != ACT_NONE else w.N
    out = torch.zeros(P, n_out, dtype=torch.float32, device=x.device)
    xf = x.to(torch.float32)
    for el in range(w.E):
        e = e_lo + el
        c, s0 = int(pk.counts[e]), int(pk.seg_start[e])
        if c == 0:
            continue
        rows = torch.arange(s0, s0 + c, device=x.device)
        xin = xf[x_index[rows].long()] if x_index is not None else xf[rows]
        y = _mm(xin, W[el])
        if bias is not None:
            y = y + bias[el]
        if act != ACT_NONE:
            g, u = _deinterleave16(y)
            y = _act(act, g, u, act_alpha, act_limit)
        out[rows] = y
    return out.to(torch.bfloat16)


def moe_combine(yp, pk: MoePacking, w, out=None, accumulate=False):
    """sum_k w[t,k] * yp[pos(t,k)] -> fp32 [T,H] (into ``out`` when given)."""
    T, K = w.shape
    pos = pk.pair_to_packed.reshape(T, K).long()
    rows = yp.to(torch.float32)[pos.clamp_min(0)]                  # [T,K,H]
    rows = rows * (pos >= 0).unsqueeze(-1) * w.unsqueeze(-1)
    y = rows.sum(dim=1)
    if out is None:
        return y
    if accumulate:
        out.add_(y.to(out.dtype))
    else:
        out.copy_(y.to(out.dtype))
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits):
    return torch.argmax(logits, dim=-1).to(torch.int32)   # first maximal index


def rep_penalty(logits, ids, penalty):
    for r in range(logits.shape[0]):
        sel = ids[r][ids[r] >= 0].long()
        if sel.numel() and float(penalty[r]) != 1.0:
            v = logits[r, sel]
            logits[r, sel] = torch.where(v > 0, v / penalty[r], v * penalty[r])
    return logits


def _xorshift(s: int) -> tuple[int, float]:
    m = (1 << 64) - 1
    s ^= s >> 12
    s ^= (s << 25) & m
    s ^= s >> 27
    z = (s * 2685821657736338717) & m
    return s, (z >> 40) / 16777216.0


def sample(logits, temperature, top_k, top_p, min_p, rng):
    """rng: int64/uint64-like tensor of xorshift states (updated in place).  Mirrors the kernel's order of cuts."""
    CAP = 256
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    for r in range(rows):
        t = float(temperature[r])
        k = int(top_k[r])
        if k <= 0 or k > CAP:
            k = CAP
        k = min(k, V)
        if t <= 0:
            out[r] = int(torch.argmax(logits[r]))
            continue
        order = torch.sort(-logits[r].to(torch.float32), stable=True).indices[:k]
        vals = logits[r, order].to(torch.float32)
        p = torch.exp((vals - vals[0]) / t)
        keep = k
        tp, mp = float(top_p[r]), float(min_p[r])
        if 0 < tp < 1:
            c = torch.cumsum(p / p.sum(), 0)
            hit = torch.nonzero(c >= tp)
            if hit.numel():
                keep = int(hit[0]) + 1
        if mp > 0:
            n = 1
            while n < keep and float(p[n]) >= mp * float(p[0]):
                n += 1
            keep = n
        state = int(rng[r]) & ((1 << 64) - 1)
        state, u = _xorshift(state)
        rng[r] = state if state < (1 << 63) else state - (1 << 64)
        u = u * float(p[:keep].sum())
        c = torch.cumsum(p[:keep], 0)
        hit = torch.nonzero(u < c)
        out[r] = int(order[int(hit[0])]) if hit.numel() else int(order[keep - 1])
    return out
