"""One decoder-only graph for the attention-based families: dense Llama / Qwen2 / Qwen3 / Mistral /
Phi-3 / Granite, Qwen3-MoE and gpt-oss (attention sinks, alternating sliding window, biased
projections, clamped SwiGLU, MXFP4 experts).  Hybrid (gated-DeltaNet) layers plug in through
``models/hybrid.py``.

The graph is config-driven instead of one class per family: the reference copies its dense
forward for every architecture (src/model/dense_transformer.cpp:381-744, gptoss.cpp:312-523,
qwen3moe.cpp) and again for every parallel form (dense_tp.cpp, gptoss_tp.cpp, qwen3moe_tp.cpp);
here parallelism is a property of the linear layers (:class:`ParallelCtx`).

Per layer the launch sequence is
  rmsnorm(+residual) -> qkv GEMM -> qkv_post (bias, QK-norm, RoPE, paged KV write) -> attention
  -> o GEMM [-> all-reduce] -> rmsnorm(+residual) -> FFN (gate|up GEMM with fused activation,
  down GEMM) or MoE (router GEMM, top-k, pack, gather, grouped GEMMs, combine) [-> all-reduce].
The residual stream is fp32, activations bf16; nothing goes back to the host inside forward.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..formats.model_config import ModelConfig
from ..ops import ACT_GEGLU, ACT_NONE, ACT_SWIGLU, ACT_SWIGLU_OAI, QuantWeight
from ..ops.weights import WFormat
from ..parallel.comm import ParallelCtx
from ..utils.rope import rope_tables

KV_BLOCK = 128


@dataclass
class ForwardBatch:
    """Device-side description of one step (prefill chunk(s), decode tokens, or a mix)."""
    ids: torch.Tensor            # int32 [T]
    positions: torch.Tensor      # int32 [T]
    slot_map: torch.Tensor       # int64 [T]  block*KV_BLOCK + offset, <0 = do not cache
    block_table: torch.Tensor    # int32 [B, max_blocks]
    seq_lens: torch.Tensor       # int32 [B]  kv length after this step
    cu_q: torch.Tensor           # int32 [B+1]
    max_q_len: int
    logit_rows: Optional[torch.Tensor] = None   # int64 rows of the T tokens that need logits (None: last of each sequence)
    state_slots: Optional[torch.Tensor] = None  # int32 [B] recurrent-state slot per sequence (hybrid models)
    state_slots_host: Optional[list] = None     # host copy of state_slots
    q_lens_host: Optional[list] = None          # host copy of per-sequence query lengths (hybrid scan scheduling)
    start_host: Optional[list] = None           # host copy of per-sequence start positions (0 = fresh state)
    want_hidden: bool = False                   # also return the pre-final-norm hidden rows (MTP)
    max_kv_len: int = 0                         # host copy of max(seq_lens); 0 = unknown (the block table's capacity is assumed)

    @property
    def T(self) -> int:
        return self.ids.numel()

    @property
    def B(self) -> int:
        return self.seq_lens.numel()


class KVCache:
    """Paged KV: per attention layer ``k, v [num_blocks, n_kv_local, KV_BLOCK, head_dim]`` bf16, or int8 with one fp32 scale
    per (block, kv head, token) row in ``ks, vs [num_blocks, n_kv_local, KV_BLOCK]`` (value = q * scale, scale = max|x| / 127).

    The reference cache is contiguous per sequence (include/ie/kv_cache.hpp:27-114) and keeps int8 rows beside it when
    ``--int8-kv`` is given (src/core/kv_cache.cpp:182-240, src/ops/attention.cpp:145-229); pages make continuous batching
    and block-level prefix sharing possible, and here the int8 rows replace the bf16 ones instead of shadowing them.
    """

    def __init__(self, n_layers: int, num_blocks: int, n_kv: int, head_dim: int, device, attn_layers: Optional[list[int]] = None,
                 dtype: str = "bf16", geometry: Optional[dict] = None):
        if dtype not in ("bf16", "int8"):
            raise ValueError(f"unknown KV cache dtype {dtype!r}")
        self.num_blocks = num_blocks
        self.block_size = KV_BLOCK
        self.dtype = dtype
        layers = attn_layers if attn_layers is not None else list(range(n_layers))
        td = torch.bfloat16 if dtype == "bf16" else torch.int8
        geo = {l: ((geometry or {}).get(l) or (n_kv, head_dim)) for l in layers}       # per layer (n_kv, head_dim): Gemma-4 mixes two
        self.k = {l: torch.zeros(num_blocks, geo[l][0], KV_BLOCK, geo[l][1], dtype=td, device=device) for l in layers}
        self.v = {l: torch.zeros(num_blocks, geo[l][0], KV_BLOCK, geo[l][1], dtype=td, device=device) for l in layers}
        self.ks = {l: torch.ones(num_blocks, geo[l][0], KV_BLOCK, dtype=torch.float32, device=device) for l in layers} if dtype == "int8" else None
        self.vs = {l: torch.ones(num_blocks, geo[l][0], KV_BLOCK, dtype=torch.float32, device=device) for l in layers} if dtype == "int8" else None

    def scales(self, layer: int):
        return (self.ks[layer], self.vs[layer]) if self.ks is not None else None

    @staticmethod
    def bytes_per_block(n_attn_layers: int, n_kv: int, head_dim: int, dtype: str = "bf16") -> int:
        per_row = head_dim * 2 if dtype == "bf16" else head_dim + 4
        return 2 * n_attn_layers * n_kv * KV_BLOCK * per_row

    def copy_blocks(self, src: list[int], dst: list[int]) -> None:
        if not src:
            return
        s = torch.tensor(src, dtype=torch.long, device=next(iter(self.k.values())).device)
        d = torch.tensor(dst, dtype=torch.long, device=s.device)
        for l in self.k:
            self.k[l][d] = self.k[l][s]
            self.v[l][d] = self.v[l][s]
            if self.ks is not None:
                self.ks[l][d] = self.ks[l][s]
                self.vs[l][d] = self.vs[l][s]


# ---------------------------------------------------------------------------------------------
class Linear:
    """y = x W^T (+b).  ``reduce`` marks a row-parallel layer whose output is a partial sum."""

    def __init__(self, w: QuantWeight, bias: Optional[torch.Tensor] = None, act: int = ACT_NONE, act_alpha: float = 1.702,
                 act_limit: float = 7.0, reduce: bool = False):
        self.w, self.bias, self.act, self.act_alpha, self.act_limit, self.reduce = w, bias, act, act_alpha, act_limit, reduce

    def __call__(self, x: torch.Tensor, par: Optional[ParallelCtx] = None, out_f32: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is not None:        # (column-parallel projections only: a caller-provided slice of a shared output)
            return ops.linear(x, self.w, bias=self.bias, act=self.act, act_alpha=self.act_alpha, act_limit=self.act_limit, out_f32=out_f32, out=out)
        if self.reduce and par is not None and par.enabled:
            # the bias of a row-parallel layer is added once, after the reduction
            if par.fused is not None and x.is_cuda:
                return par.fused.linear_all_reduce(x, self.w, self.bias)
            y = par.all_reduce(ops.linear(x, self.w, out_f32=True))
            return y if self.bias is None else y + self.bias
        return ops.linear(x, self.w, bias=self.bias, act=self.act, act_alpha=self.act_alpha, act_limit=self.act_limit, out_f32=out_f32)


class MultiLinear:
    """Column-concatenation of linears whose weights have different storage formats (e.g. Q4_K q/k with Q6_K v)."""

    def __init__(self, parts: list[Linear]):
        self.parts = parts
        self.widths = [p.w.N // 2 if p.act != ACT_NONE else p.w.N for p in parts]

    def __call__(self, x, par=None, out_f32=False):
        # every part writes its own column slice of one output (no concatenation pass)
        out = torch.empty(x.shape[0], sum(self.widths), dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
        lo = 0
        for p, n in zip(self.parts, self.widths):
            p(x, par, out_f32, out=out[:, lo:lo + n])
            lo += n
        return out


def _fuse_rows(ws: list[QuantWeight], biases: list[Optional[torch.Tensor]]):
    if all(w.fmt == ws[0].fmt for w in ws) and ws[0].fmt != WFormat.EXL3:
        b = None
        if any(bb is not None for bb in biases):
            b = torch.cat([bb if bb is not None else torch.zeros(w.N, device=w.device) for w, bb in zip(ws, biases)])
        return Linear(QuantWeight.cat_rows(ws), b)
    return MultiLinear([Linear(w, b) for w, b in zip(ws, biases)])


def unpermute_llama_qk(w: QuantWeight, n_heads: int, head_dim: int) -> QuantWeight:
    """GGUF ``llama`` files store Q/K rows interleaved for pairwise RoPE; the kernels rotate NEOX
    half-splits, so rows are regrouped: dest h*hd + b*hd/2 + k  <-  src h*hd + 2k + b
    (src/model/dense_transformer.cpp:24-32,130-137)."""
    hd = head_dim
    k = torch.arange(hd // 2)
    src = torch.cat([2 * k, 2 * k + 1])                       # b = 0 block then b = 1 block
    idx = (torch.arange(n_heads).unsqueeze(1) * hd + src.unsqueeze(0)).reshape(-1)
    return w.select_rows(idx)


class AttentionBlock:
    def __init__(self, cfg: ModelConfig, layer: int, src, par: ParallelCtx, prefix: Optional[str] = None, q_gate: bool = False):
        c = cfg
        p = prefix or f"blk.{layer}"
        if c.arch == "gemma4":           # per-layer head geometry: the rest of this constructor sees a config of this layer's shape
            from dataclasses import replace
            hd_l, n_kv_l, n_rot_l, _ = c.layer_geometry(layer)
            c = replace(c, head_dim=hd_l, n_kv_heads=n_kv_l, n_rot=n_rot_l)
        hd, H = c.head_dim, c.hidden
        tp = par.world if par.mode == "tp" else 1
        self.layer = layer
        self.q_gate = q_gate
        self.n_q = c.n_heads // tp
        if c.n_heads % tp:
            raise ValueError(f"{c.n_heads} attention heads do not split over {tp} ranks")
        # KV heads: shard when they divide, otherwise each rank keeps the one head its query heads use
        if c.n_kv_heads >= tp:
            if c.n_kv_heads % tp:
                raise ValueError(f"{c.n_kv_heads} KV heads do not split over {tp} ranks")
            self.n_kv = c.n_kv_heads // tp
            kv_lo = par.rank * self.n_kv if tp > 1 else 0
        else:
            self.n_kv = 1
            kv_lo = (par.rank * c.n_kv_heads) // tp
        q_lo = (par.rank * self.n_q) if tp > 1 else 0
        q_rows_per_head = hd * (2 if q_gate else 1)

        if c.arch == "phi3" and not src.has(f"{p}.attn_q.weight"):
            # Phi-3 files keep one fused attn_qkv matrix: q rows, then k rows, then v rows
            nq_rows, nkv_rows = c.n_heads * hd, c.n_kv_heads * hd
            fused = src.matrix(f"{p}.attn_qkv.weight", nq_rows + 2 * nkv_rows, H)
            wq, wk, wv = fused.slice_rows(0, nq_rows), fused.slice_rows(nq_rows, nq_rows + nkv_rows), fused.slice_rows(nq_rows + nkv_rows, nq_rows + 2 * nkv_rows)
        else:
            wq = src.matrix(f"{p}.attn_q.weight", c.n_heads * q_rows_per_head, H)
            wk = src.matrix(f"{p}.attn_k.weight", c.n_kv_heads * hd, H)
            has_v = True
            if c.arch == "gemma4":       # files simply lack attn_v on the global layers; random-init graphs decide by the pattern
                has_v = src.has(f"{p}.attn_v.weight") if getattr(src, "r", None) is not None else bool(c.layer_swa[layer])
            if not has_v:
                wv = wk                  # V is the raw K projection (src/model/gemma4.cpp:178-183,660)
            else:
                wv = src.matrix(f"{p}.attn_v.weight", c.n_kv_heads * hd, H)
        if c.arch == "llama" and getattr(src, "r", None) is not None and wq.fmt != WFormat.EXL3:
            # (imported EXL3 layers keep the Hugging Face row order, which is the half-split one: src/model/dense_transformer.cpp:165-212)
            wq, wk = unpermute_llama_qk(wq, c.n_heads, hd), unpermute_llama_qk(wk, c.n_kv_heads, hd)
        has_bias = c.arch in ("qwen2", "gpt-oss") and src.has(f"{p}.attn_q.bias")
        bq = src.vector(f"{p}.attn_q.bias", c.n_heads * q_rows_per_head) if has_bias else None
        bk = src.vector(f"{p}.attn_k.bias", c.n_kv_heads * hd) if has_bias else None
        bv = src.vector(f"{p}.attn_v.bias", c.n_kv_heads * hd) if has_bias else None
        sl = lambda w, lo, n: w if (lo == 0 and n == w.N) else w.slice_rows(lo, lo + n)
        sb = lambda b, lo, n: None if b is None else b[lo:lo + n].contiguous()
        ws = [sl(wq, q_lo * q_rows_per_head, self.n_q * q_rows_per_head), sl(wk, kv_lo * hd, self.n_kv * hd), sl(wv, kv_lo * hd, self.n_kv * hd)]
        bs = [sb(bq, q_lo * q_rows_per_head, self.n_q * q_rows_per_head), sb(bk, kv_lo * hd, self.n_kv * hd), sb(bv, kv_lo * hd, self.n_kv * hd)]
        self.qkv = _fuse_rows(ws, bs)
        wo = src.matrix(f"{p}.attn_output.weight", H, c.n_heads * hd)
        bo = src.vector(f"{p}.attn_output.bias", H) if (c.arch == "gpt-oss" and src.has(f"{p}.attn_output.bias")) else None
        if tp > 1:
            wo = wo.slice_k(q_lo * hd, (q_lo + self.n_q) * hd, requant=True)
        self.o = Linear(wo, bo, reduce=tp > 1)
        qk_norm = c.arch in ("qwen3", "qwen3moe", "qwen3next", "qwen35", "qwen35moe", "gemma4") and src.has(f"{p}.attn_q_norm.weight")
        self.v_norm = c.arch == "gemma4"       # weightless RMS norm on V (src/model/gemma4.cpp:663)
        self.q_norm = src.vector(f"{p}.attn_q_norm.weight", hd) if qk_norm else None
        self.k_norm = src.vector(f"{p}.attn_k_norm.weight", hd) if qk_norm else None
        self.sinks = None
        if c.arch == "gpt-oss":
            s = src.vector(f"{p}.attn_sinks.weight", c.n_heads)
            self.sinks = s[q_lo:q_lo + self.n_q].contiguous()
        self.window = c.layer_window(layer)
        self.scale = c.attention_scale if c.attention_scale > 0 else 1.0 / math.sqrt(hd)
        self.hd, self.n_rot, self.eps = hd, c.n_rot, c.rms_eps
        self.norm_one_plus_w = c.arch in ("qwen35", "qwen35moe")      # Qwen3-Next files store 1 + w already

    def __call__(self, h: torch.Tensor, fb: ForwardBatch, kv: KVCache, rope, par: ParallelCtx) -> torch.Tensor:
        return self.attend(self.qkv(h), fb, kv, rope, par)

    def attend(self, qkv: torch.Tensor, fb: ForwardBatch, kv: KVCache, rope, par: ParallelCtx) -> torch.Tensor:
        """Everything after the qkv projection: head epilogue + cache write, attention, output projection."""
        q, gate = ops.qkv_post(qkv, None, self.q_norm, self.k_norm, fb.positions, rope[0], rope[1], fb.slot_map, kv.k[self.layer],
                               kv.v[self.layer], self.n_q, self.n_kv, self.hd, self.n_rot, q_gate=self.q_gate,
                               norm_one_plus_w=self.norm_one_plus_w, eps=self.eps, kv_scales=kv.scales(self.layer),
                               **({"v_norm": True} if self.v_norm else {}))
        a = ops.attention(q, kv.k[self.layer], kv.v[self.layer], fb.block_table, fb.seq_lens, fb.cu_q, fb.max_q_len, sinks=self.sinks,
                          window=self.window, scale=self.scale, kv_scales=kv.scales(self.layer), max_kv_len=fb.max_kv_len)
        a = a.reshape(a.shape[0], self.n_q * self.hd)
        if gate is not None:
            a = ops.sigmoid_mul(a, gate.reshape(a.shape))
        return self.o(a, par)


def _attn_gathered(self, sc, T: int, gbuf: int, fb: ForwardBatch, kv: KVCache, rope, par: ParallelCtx):
    """Row-sharded prefill: qkv on the gathered rows (all-gather -> GEMM), attention over this rank's heads, and the output
    projection with the reduce-scatter epilogue (each row's partial goes to the rank that owns the row)."""
    qkv = sc.linear_gathered(self.qkv, T, gbuf)
    q, gate = ops.qkv_post(qkv, None, self.q_norm, self.k_norm, fb.positions, rope[0], rope[1], fb.slot_map, kv.k[self.layer],
                           kv.v[self.layer], self.n_q, self.n_kv, self.hd, self.n_rot, q_gate=self.q_gate,
                           norm_one_plus_w=self.norm_one_plus_w, eps=self.eps, kv_scales=kv.scales(self.layer),
                           **({"v_norm": True} if self.v_norm else {}))
    a = ops.attention(q, kv.k[self.layer], kv.v[self.layer], fb.block_table, fb.seq_lens, fb.cu_q, fb.max_q_len, sinks=self.sinks,
                      window=self.window, scale=self.scale, kv_scales=kv.scales(self.layer), max_kv_len=fb.max_kv_len)
    a = a.reshape(a.shape[0], self.n_q * self.hd)
    if gate is not None:
        a = ops.sigmoid_mul(a, gate.reshape(a.shape))
    return par.fused.linear_all_reduce(a, self.o.w, self.o.bias, rs_rows=T // par.world)


AttentionBlock.forward_gathered = _attn_gathered


class DenseFFN:
    def __init__(self, cfg: ModelConfig, layer: int, src, par: ParallelCtx, prefix: Optional[str] = None, act: int = ACT_SWIGLU,
                 ffn: Optional[int] = None, suffix: str = ""):
        p = prefix or f"blk.{layer}"
        H, F = cfg.hidden, ffn or cfg.ffn
        tp = par.world if par.mode == "tp" else 1
        if cfg.arch == "phi3" and not src.has(f"{p}.ffn_gate{suffix}.weight"):
            up2 = src.matrix(f"{p}.ffn_up{suffix}.weight", 2 * F, H)            # fused gate|up rows
            g, u = up2.slice_rows(0, F), up2.slice_rows(F, 2 * F)
        else:
            g = src.matrix(f"{p}.ffn_gate{suffix}.weight", F, H)
            u = src.matrix(f"{p}.ffn_up{suffix}.weight", F, H)
        d = src.matrix(f"{p}.ffn_down{suffix}.weight", H, F)
        if tp > 1:
            gran = max(d.k_granule(), 16)
            if F % gran or (F // gran) < tp:
                gran = 32 if F % 32 == 0 else 16          # finer than the weight's blocks: the shard is re-encoded
            lo, hi = _even_chunks(F, tp, gran)[par.rank]
            g, u, d = g.slice_rows(lo, hi), u.slice_rows(lo, hi), d.slice_k(lo, hi, requant=True)
        if g.fmt == u.fmt and g.fmt != WFormat.EXL3:
            self.gate_up = Linear(QuantWeight.interleave_gate_up(g, u), act=act)
            self.split = None
        else:
            self.gate_up = None
            self.split = (Linear(g), Linear(u))
            self.act = act
        self.down = Linear(d, reduce=tp > 1)

    def __call__(self, h, par):
        if self.gate_up is not None:
            a = self.gate_up(h)
        else:
            g, u = self.split[0](h), self.split[1](h)
            F = g.shape[1]
            il = torch.cat([g.reshape(-1, F // 16, 16), u.reshape(-1, F // 16, 16)], dim=2).reshape(-1, 2 * F)
            a = ops.glu(il.contiguous(), self.act)
        return self.down(a, par)


def _ffn_gathered(self, sc, T: int, gbuf: int, par: ParallelCtx):
    if self.gate_up is not None:
        a = sc.linear_gathered(self.gate_up, T, gbuf)
    else:
        g, u = sc.linear_gathered(self.split[0], T, gbuf), sc.linear_gathered(self.split[1], T, gbuf)
        F = g.shape[1]
        il = torch.cat([g.reshape(-1, F // 16, 16), u.reshape(-1, F // 16, 16)], dim=2).reshape(-1, 2 * F)
        a = ops.glu(il.contiguous(), self.act)
    return par.fused.linear_all_reduce(a, self.down.w, self.down.bias, rs_rows=T // par.world)


DenseFFN.forward_gathered = _ffn_gathered


def _even_chunks(n: int, parts: int, gran: int) -> list[tuple[int, int]]:
    """Split n (a multiple of gran) into `parts` contiguous ranges on gran boundaries, sizes differing by <= gran."""
    blocks = n // gran
    base, extra = divmod(blocks, parts)
    out, lo = [], 0
    for r in range(parts):
        sz = (base + (1 if r < extra else 0)) * gran
        out.append((lo, lo + sz))
        lo += sz
    return out


class MoEFFN:
    """Router -> top-k -> experts -> weighted combine, expert-parallel over the ranks of ``par``.

    Every rank sees every token (activations are replicated under tensor parallelism), packs only
    the pairs routed to its own experts and contributes a partial sum that the caller reduces.
    """

    MXF4_TENSOR_CORE = True      # class switch (tests compare against the bf16-activation path by turning it off)
    EXPERT_TP = False            # True: split every expert's FFN width over the ranks even when the expert count divides (tests)
    MXF4_PAIR_MAX_TOKENS = 8     # up to this many tokens every (token, expert) pair is its own tile: no packing pass
    DOWN_KSPLIT = 3              # one-token decode: K ranges of the down projection (their partial rows are summed by the combine)

    def __init__(self, cfg: ModelConfig, layer: int, src, par: ParallelCtx, act: int, with_bias: bool, prefix: Optional[str] = None):
        c = cfg
        p = prefix or f"blk.{layer}"
        H, F, E = c.hidden, c.expert_ffn, c.n_experts
        ep = par.world if par.mode == "tp" else 1
        # Experts are sharded whole (expert parallelism) when their count divides by the ranks.  Otherwise (or with EXPERT_TP) every
        # rank keeps all experts and a slice of each one's FFN width, cut on the 32-element blocks of the quantised formats and not
        # necessarily even (src/model/gptoss_tp.cpp:343-354 in the reference): gate / up rows [lo, hi), the matching input columns of
        # down, the down bias on rank 0 only; every rank then holds a partial sum for every pair, reduced like any row-parallel output.
        self.expert_tp = ep > 1 and (E % ep != 0 or self.EXPERT_TP)
        self.E, self.K = E, c.n_experts_used
        self.e_lo, self.e_hi = (par.rank * (E // ep), (par.rank + 1) * (E // ep)) if (ep > 1 and not self.expert_tp) else (0, E)
        rng = (self.e_lo, self.e_hi)
        f_lo, f_hi = 0, F
        if self.expert_tp:
            if F % 32 or F // 32 < ep:
                raise ValueError(f"expert FFN width {F} cannot be cut into {ep} slices of whole 32-element blocks")
            f_lo, f_hi = _even_chunks(F, ep, 32)[par.rank]
        rw = src.matrix(f"{p}.ffn_gate_inp.weight", E, H)
        self.router = Linear(rw if rw.fmt == ops.WFormat.BF16 else QuantWeight(**_as_bf16(rw)))
        self.router_bias = src.vector(f"{p}.ffn_gate_inp.bias", E) if with_bias else None
        if c.arch == "gemma4":           # one bank [E, gate rows | up rows, H] (src/model/gemma4.cpp:267-289)
            gu = src.matrix(f"{p}.ffn_gate_up_exps.weight", 2 * F, H, E, experts=rng)
            g, u = gu.slice_rows(0, F), gu.slice_rows(F, 2 * F)
            del gu
        else:
            g = src.matrix(f"{p}.ffn_gate_exps.weight", F, H, E, experts=rng)
            u = src.matrix(f"{p}.ffn_up_exps.weight", F, H, E, experts=rng)
        d = src.matrix(f"{p}.ffn_down_exps.weight", H, F, E, experts=rng)
        if self.expert_tp:
            g, u, d = g.slice_rows(f_lo, f_hi), u.slice_rows(f_lo, f_hi), d.slice_k(f_lo, f_hi, requant=True)
        # MXFP4 banks on a GPU run on the block-scaled tensor-core kernel: gate / up / down stay three banks in its tiled layout
        self.mx = None
        # all-MXFP4 expert banks multiply MXFP8 activations (e4m3 + a power-of-two scale per 32): the arithmetic of the block-scaled
        # tensor-core kernel, and the arithmetic the CPU path restates so that both produce the same numbers
        self.a8 = g.fmt == u.fmt == d.fmt == ops.WFormat.MXFP4 and act in (ACT_SWIGLU, ACT_SWIGLU_OAI) and self.MXF4_TENSOR_CORE
        if g.p0.is_cuda and self.a8:
            from ..ops.weights import to_mxf4_tiles
            self.mx = (to_mxf4_tiles(g, u), to_mxf4_tiles(d))
            self.gate_up = self.down = None
        else:
            self.gate_up = QuantWeight.interleave_gate_up(g, u)
            self.down = d
        del g, u, d
        # banks past the device's expert budget live in host memory and are staged per forward (models/spill.py)
        self._spill = None
        from . import spill as _spill_mod
        sp = _spill_mod.active()
        if sp is not None:
            banks = list(self.mx) if self.mx is not None else [self.gate_up, self.down]
            if not sp.admit(sum(b.nbytes for b in banks)):
                self._spill = (sp, [sp.to_host(i, b) for i, b in enumerate(banks)])
                self._stage_banks()
        self.expert_scale = None         # optional per-expert factor on the down projection's output, folded into the routing weight
        self.gu_bias = self.down_bias = self.g_bias = self.u_bias = None
        if with_bias:
            gb = src.table(f"{p}.ffn_gate_exps.bias", (E, F))[self.e_lo:self.e_hi, f_lo:f_hi]
            ub = src.table(f"{p}.ffn_up_exps.bias", (E, F))[self.e_lo:self.e_hi, f_lo:f_hi]
            F = f_hi - f_lo
            n = self.e_hi - self.e_lo
            if self.mx is not None:
                self.g_bias, self.u_bias = gb.contiguous(), ub.contiguous()
            else:
                self.gu_bias = torch.cat([gb.reshape(n, F // 16, 16), ub.reshape(n, F // 16, 16)], dim=2).reshape(n, 2 * F).contiguous()
            self.down_bias = src.table(f"{p}.ffn_down_exps.bias", (E, H))[self.e_lo:self.e_hi].contiguous()
            if self.expert_tp and par.rank != 0:
                self.down_bias = torch.zeros_like(self.down_bias)      # the bias joins the reduced sum once
        self.act = act
        self.reduce = ep > 1
        self.group_gemv_max_tokens = 0   # > 0: batches of up to that many tokens take the expert-major GEMV path
        self.shared = None          # optional always-on expert (hybrid families): its partial joins the sum before the reduction
        self._arange = {}

    def _stage_banks(self) -> None:
        """Spilled layer: copy the banks from host memory into the shared staging area and point the layer at them."""
        sp, host = self._spill
        banks = [sp.fetch(i, b) for i, b in enumerate(host)]
        if self.mx is not None:
            self.mx = (banks[0], banks[1])
        else:
            self.gate_up, self.down = banks

    def __call__(self, h: torch.Tensor, par: ParallelCtx, router_h: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns this rank's fp32 contribution [T, H] (already reduced when EP > 1).  ``router_h``: the router's own input
        when it differs from the experts' (Gemma-4)."""
        if self._spill is not None:
            self._stage_banks()
        T = h.shape[0]
        pre = None
        ksplit = 1
        if not isinstance(router_h, tuple):
            logits = self.router(h if router_h is None else router_h, out_f32=True)
        if isinstance(router_h, tuple):
            # decode: the router GEMV's launch has already routed and quantised the rows (ops.cuda.gemv_norm)
            idx, w, xq, sfx = router_h
            pre = (xq, sfx)
            ksplit = w.shape[1] // self.K
        elif self.mx is not None and T <= self.MXF4_PAIR_MAX_TOKENS:
            # decode: routing and the MXFP8 rounding of the token rows share one launch
            from ..ops.cuda import moe_route_quant
            # one token on one rank: the down projection has too few (pair, column block) items for the chip and splits K
            if T * self.K <= 4 and not self.reduce and self.shared is None and self.expert_scale is None:
                from ..ops.cuda import mxf4_ksplit
                ksplit = mxf4_ksplit(self.mx[1].K, self.DOWN_KSPLIT)
            idx, w, xq, sfx = moe_route_quant(logits, self.router_bias, self.K, h, w_copies=ksplit)
            pre = (xq, sfx)
        else:
            idx, w = ops.moe_route(logits, self.router_bias, self.K, True)
        if self.expert_scale is not None:
            w = w * self.expert_scale[idx.long()]
        local = self.e_hi - self.e_lo
        # expert parallelism on the peer-memory path: the combine writes its partial into every rank's inbox itself
        fuse_push = self.reduce and par.fused is not None and h.is_cuda and self.shared is None
        if self.mx is not None:
            y, p2p = self._mx_experts(h, idx, pre, ksplit)
            if fuse_push:
                return par.fused.moe_combine_push(y, p2p, w)
            if self.shared is None and not self.reduce and self.K <= 32:
                # single rank: the weighted sum is formed inside the residual add + norm that consumes it
                from ..ops.cuda import CombineDelta
                return CombineDelta(y, p2p, w.contiguous())
            out = ops.moe_combine(y, ops.ref.MoePacking(None, None, None, p2p, None, None, y.shape[0], self.K), w)
        elif self.a8:
            # CPU restatement of the block-scaled path: same rounding points, fp32 math
            q8 = lambda t: ops.ref.mxfp8_roundtrip(t).to(torch.bfloat16)
            slot_e = idx.reshape(-1)
            a = ops.expert_gemv(q8(h), self.gate_up, slot_e, x_div=self.K, bias=self.gu_bias, act=self.act, e_lo=self.e_lo)
            y = ops.expert_gemv(q8(a), self.down, slot_e, x_div=1, bias=self.down_bias, e_lo=self.e_lo)
            pk = ops.ref.MoePacking(None, None, None, torch.arange(T * self.K, dtype=torch.int32, device=h.device), None, None, T * self.K, self.K)
            out = ops.moe_combine(y, pk, w)
        elif T <= 8:
            # decode: one GEMV slot per (token, expert) pair, weights streamed once per pair; under expert
            # parallelism the slots of experts that live on other ranks contribute zero rows here
            slot_e = idx.reshape(-1)
            a = ops.expert_gemv(h, self.gate_up, slot_e, x_div=self.K, bias=self.gu_bias, act=self.act, e_lo=self.e_lo)
            y = ops.expert_gemv(a, self.down, slot_e, x_div=1, bias=self.down_bias, e_lo=self.e_lo)
            key = (T, h.device)
            if key not in self._arange:
                pk = ops.ref.MoePacking(None, None, torch.zeros(1, dtype=torch.int32, device=h.device),
                                        torch.arange(T * self.K, dtype=torch.int32, device=h.device), None, None, T * self.K, self.K)
                self._arange[key] = pk
            if fuse_push:
                return par.fused.moe_combine_push(y, self._arange[key].pair_to_packed, w)
            out = ops.moe_combine(y, self._arange[key], w)
        elif T <= self.group_gemv_max_tokens and T * self.K <= 8 * local:
            # expert-major GEMV over a compact packing: every local expert streams its weights once against all of its rows (token
            # rows are read in place through the packing's index: no gather, no tile padding).  Measured slower than the grouped
            # tensor-core GEMM for gpt-oss-120b at 64 concurrent sequences (75 vs 61 ms per step), so it is off by default.
            pk = ops.moe_pack(idx, self.E, self.e_lo, self.e_hi, tile=1)
            a = ops.expert_group_gemv(h, self.gate_up, pk, x_index=pk.packed_token, bias=self.gu_bias, act=self.act, e_lo=self.e_lo)
            y = ops.expert_group_gemv(a, self.down, pk, bias=self.down_bias, e_lo=self.e_lo)
            if fuse_push:
                return par.fused.moe_combine_push(y, pk.pair_to_packed, w)
            out = ops.moe_combine(y, pk, w)
        else:
            pk = ops.moe_pack(idx, self.E, self.e_lo, self.e_hi)
            xp = ops.moe_gather(h, pk)
            te = pk.tile_expert - self.e_lo if self.e_lo else pk.tile_expert
            a = ops.grouped_linear(xp, self.gate_up, te, pk.num_tiles, bias=self.gu_bias, act=self.act)
            y = ops.grouped_linear(a, self.down, te, pk.num_tiles, bias=self.down_bias)
            if fuse_push:
                return par.fused.moe_combine_push(y, pk.pair_to_packed, w)
            out = ops.moe_combine(y, pk, w)
        if self.shared is not None:
            out = self.shared.add_into(out, h)
        if self.reduce:
            out = par.fused.push(out) if (par.fused is not None and out.is_cuda) else par.all_reduce(out)
        return out


def _mx_experts(self, h: torch.Tensor, idx: torch.Tensor, pre=None, ksplit: int = 1):
    """Expert projections on the block-scaled MXFP4 kernel.  Returns (y bf16 [rows, H], pair_to_packed int32 [T*K]).  ``pre``: the
    pair-mode (xq, sfx) when the router launch has already quantised the rows.  ``ksplit`` (pair mode): the down projection leaves
    that many partial rows per pair, and pair_to_packed lists them all ([T, ksplit, K])."""
    from ..ops import cuda as K_
    gate_up, down = self.mx
    T = h.shape[0]
    ep = dict(e_lo=self.e_lo)
    if T <= self.MXF4_PAIR_MAX_TOKENS:
        # decode: pair i = (token i // K, slot i % K) is tile i with one live row; no sort, no gather
        n = T * self.K
        te = idx.reshape(-1)
        xq, sfx = pre if pre is not None else K_.moe_quant(h, n, n, 1, x_div=self.K)
        aq, sfa = K_.mxf4_gemm(gate_up, xq, sfx, te, n, 1, default_valid=1, bias0=self.g_bias, bias1=self.u_bias, act=self.act, **ep)
        y = K_.mxf4_gemm(down, aq, sfa, te, n, 1, default_valid=1, bias0=self.down_bias, zero_out=self.reduce, ksplit=ksplit, **ep)
        key = (T, ksplit, h.device)
        if key not in self._arange:
            # pair (t, k) sits at row t * K + k of every K range's block of n rows
            base = torch.arange(n, dtype=torch.int32, device=h.device).reshape(T, 1, self.K)
            off = (torch.arange(ksplit, dtype=torch.int32, device=h.device) * n).reshape(1, ksplit, 1)
            self._arange[key] = (base + off).reshape(-1).contiguous()
        return y, self._arange[key]
    pk = ops.moe_pack(idx, self.E, self.e_lo, self.e_hi)
    mt = pk.tile_expert.numel()
    tiles = dict(tile_valid=pk.tile_valid, num_tiles=pk.num_tiles)
    xq, sfx = K_.moe_quant(h, pk.max_rows, mt, 128, src_index=pk.packed_token, row_limit=pk.num_tiles)
    aq, sfa = K_.mxf4_gemm(gate_up, xq, sfx, pk.tile_expert, mt, 128, bias0=self.g_bias, bias1=self.u_bias, act=self.act, **tiles, **ep)
    y = K_.mxf4_gemm(down, aq, sfa, pk.tile_expert, mt, 128, bias0=self.down_bias, **tiles, **ep)
    return y, pk.pair_to_packed


MoEFFN._mx_experts = _mx_experts


def _moe_sharded(self, h: torch.Tensor, sc) -> torch.Tensor:
    """Row-sharded prefill: this rank routes only its own rows ``h`` [R, H], the rows travel as MXFP8 to the ranks that own their
    experts, and the expert outputs come back to be summed here.  Returns the fp32 contribution [R, H]."""
    from ..ops import cuda as K_
    gate_up, down = self.mx
    logits = self.router(h, out_f32=True)
    idx, w = ops.moe_route(logits, self.router_bias, self.K, True)
    if self.expert_scale is not None:
        w = w * self.expert_scale[idx.long()]
    xq, sfx, plan = sc.dispatch(h, idx)
    tiles = dict(tile_valid=plan.tile_valid, num_tiles=plan.num_tiles, e_lo=self.e_lo)
    aq, sfa = K_.mxf4_gemm(gate_up, xq, sfx, plan.tile_expert, plan.max_tiles, 128, bias0=self.g_bias, bias1=self.u_bias, act=self.act, **tiles)
    y = K_.mxf4_gemm(down, aq, sfa, plan.tile_expert, plan.max_tiles, 128, bias0=self.down_bias, **tiles)
    return sc.combine(y, plan, w)


MoEFFN.forward_sharded = _moe_sharded


def _as_bf16(w: QuantWeight) -> dict:
    d = w.dequantize(torch.bfloat16)
    return dict(fmt=ops.WFormat.BF16, N=w.N, K=w.K, E=w.E, p0=d.contiguous())


# ---------------------------------------------------------------------------------------------
class TransformerModel:
    def __init__(self, cfg: ModelConfig, src, device, par: Optional[ParallelCtx] = None, max_ctx: int = 8192):
        self.cfg, self.device = cfg, torch.device(device)
        self.par = par or ParallelCtx()
        c, par = cfg, self.par
        self.max_ctx = max_ctx
        tp = par.world if par.mode == "tp" else 1
        # layer split (pipeline) plan: contiguous layer ranges, embedding on the first rank, head on the last
        # (LayerPlan::contiguous, src/model/dense_split.cpp:24-33)
        self.pp = par.mode == "pp" and par.world > 1
        self.tap = None          # optional callable(layer, mixer_out, ffn_out, residual) used by the layer-dump tool
        self.layer_lo, self.layer_hi = ((par.rank * c.n_layers) // par.world, ((par.rank + 1) * c.n_layers) // par.world) if self.pp else (0, c.n_layers)
        self.first_stage, self.last_stage = (not self.pp or par.rank == 0), (not self.pp or par.rank == par.world - 1)
        self.tied = not src.has("output.weight") or c.tie_embeddings
        self.embed_w = src.matrix("token_embd.weight", c.vocab, c.hidden) if (self.first_stage or (self.last_stage and self.tied)) else None
        head = None
        if self.last_stage:
            head = self.embed_w if self.tied else src.matrix("output.weight", c.vocab, c.hidden)
        self.vocab_lo, self.vocab_hi = 0, c.vocab
        if tp > 1:
            lo, hi = _even_chunks(c.vocab, tp, 16)[par.rank] if c.vocab % (16 * tp) == 0 else (0, c.vocab)
            if (lo, hi) != (0, c.vocab):
                head = head.slice_rows(lo, hi)
                self.vocab_lo, self.vocab_hi = lo, hi
        self.lm_head = Linear(head) if head is not None else None
        self.out_norm = src.vector("output_norm.weight", c.hidden)
        ff = src.vector("rope_freqs.weight", c.n_rot // 2) if (c.arch == "llama" and getattr(src, "r", None) is not None and src.has("rope_freqs.weight")) else None
        self.rope = rope_tables(max_ctx, c.n_rot, c.rope_theta, ff, c.rope_scaling_type, c.rope_scaling_factor, c.rope_orig_ctx,
                                c.yarn_beta_fast, c.yarn_beta_slow, device=self.device)
        self.one_plus_w = c.arch in ("qwen35", "qwen35moe")
        self.layer_ids = list(range(self.layer_lo, self.layer_hi))
        self.layers = [self._build_layer(l, src) for l in self.layer_ids]
        self.attn_layers = [l for l in self.layer_ids if c.layer_is_full_attention(l)]
        self.n_kv_local = next((L["attn"].n_kv for L in self.layers if "attn" in L), 0)

    # ---- construction
    def _build_layer(self, l: int, src) -> dict:
        c, par = self.cfg, self.par
        p = f"blk.{l}"
        L = {"attn_norm": src.vector(f"{p}.attn_norm.weight", c.hidden)}
        L["attn"] = AttentionBlock(c, l, src, par)
        post = f"{p}.post_attention_norm.weight" if c.arch in ("gpt-oss",) else f"{p}.ffn_norm.weight"
        L["ffn_norm"] = src.vector(post, c.hidden)
        if c.arch == "gpt-oss":
            L["moe"] = MoEFFN(c, l, src, par, ACT_SWIGLU_OAI, with_bias=True)
        elif c.arch == "qwen3moe":
            L["moe"] = MoEFFN(c, l, src, par, ACT_SWIGLU, with_bias=False)
        else:
            L["ffn"] = DenseFFN(c, l, src, par)
        return L

    def new_kv_cache(self, num_blocks: int, dtype: str = "bf16") -> KVCache:
        return KVCache(self.cfg.n_layers, num_blocks, self.n_kv_local, self.cfg.head_dim, self.device, self.attn_layers, dtype=dtype)

    def weight_bytes(self) -> int:
        n = (self.embed_w.nbytes if self.embed_w is not None else 0) + (0 if (self.tied or self.lm_head is None) else self.lm_head.w.nbytes)
        for L in self.layers:
            for v in L.values():
                n += _bytes_of(v)
        return n

    # ---- forward
    def forward(self, fb: ForwardBatch, kv: KVCache, state=None) -> torch.Tensor:
        """Returns fp32 logits [rows, vocab] for ``fb.logit_rows`` (default: last token of each sequence)."""
        if self.pp:
            return self._forward_pipeline(fb, kv, state)
        c = self.cfg
        if self._can_shard(fb, state):
            return self._forward_sharded(fb, kv)
        x = ops.embed(self.embed_w, fb.ids, c.embedding_scale)
        x, delta = self._run_layers(x, None, fb, kv, state)
        return self._head(x, delta, fb)

    # ---- row-sharded prefill (tensor / expert parallel ranks each keep T / W rows of the residual stream)
    def _can_shard(self, fb: ForwardBatch, state) -> bool:
        par = self.par
        sc = getattr(par, "sharded", None)
        if sc is None or par.fused is None or state is not None or self.tap is not None or fb.want_hidden or type(self) is not TransformerModel:
            return False
        if not sc.can_shard(fb.T) or fb.T < self.SHARD_MIN_TOKENS:
            return False
        return all(("moe" not in L) or (L["moe"].mx is not None and L["moe"].shared is None and not L["moe"].expert_tp and L["moe"]._spill is None)
                   for L in self.layers)

    SHARD_MIN_TOKENS = 512

    def _forward_sharded(self, fb: ForwardBatch, kv: KVCache) -> torch.Tensor:
        """Prefill with the residual stream sharded by rows: per layer one all-gather (fused into the qkv GEMM's operand load), one
        reduce-scatter (the output projection's epilogue) and, for expert layers, an all-to-all of MXFP8 rows and bf16 results; dense
        FFN layers take a second gather / scatter pair.  Norms, routing, packing and quantisation run on T / W rows."""
        c, par = self.cfg, self.par
        sc = par.sharded
        T = fb.T
        row0, R = sc.rows(T)
        x = ops.embed(self.embed_w, fb.ids[row0:row0 + R].contiguous(), c.embedding_scale)
        rs = c.residual_scale
        nk = dict(one_plus_w=self.one_plus_w, delta_scale=rs)
        delta = None
        for L in self.layers:
            _, g = sc.norm(x, L["attn_norm"], c.rms_eps, T, delta=delta, gather=True, **nk)
            a = L["attn"].forward_gathered(sc, T, g, fb, kv, self.rope, par)
            if "moe" in L:
                h2, _ = sc.norm(x, L["ffn_norm"], c.rms_eps, T, delta=a, want_local=True, **nk)
                delta = L["moe"].forward_sharded(h2, sc)
            else:
                _, g2 = sc.norm(x, L["ffn_norm"], c.rms_eps, T, delta=a, gather=True, **nk)
                delta = L["ffn"].forward_gathered(sc, T, g2, par)
        sc.norm(x, self.out_norm, c.rms_eps, T, delta=delta, **nk)            # folds the last delta into the residual rows
        # the rows that need logits, replicated: each rank contributes the ones it owns
        rows = fb.logit_rows if fb.logit_rows is not None else (fb.cu_q[1:].long() - 1)
        local = rows.long() - row0
        mine = ((local >= 0) & (local < R)).unsqueeze(-1)
        xr = torch.where(mine, x.index_select(0, local.clamp(0, R - 1)), torch.zeros((), dtype=x.dtype, device=x.device))
        if par.world > 1:
            par.all_reduce(xr)
        hn = ops.rmsnorm(xr, self.out_norm, c.rms_eps, one_plus_w=self.one_plus_w)
        logits = self.lm_head(hn, out_f32=True)
        if self.vocab_hi - self.vocab_lo != c.vocab:
            logits = par.all_gather_cols(logits)
        if c.logit_scale != 1.0:
            logits = logits * c.logit_scale
        if c.final_logit_softcap > 0:
            logits = torch.tanh(logits / c.final_logit_softcap) * c.final_logit_softcap
        return logits

    # Decode with the norms inside the GEMVs that consume them (ops.cuda.gemv_norm).  Measured on gpt-oss-120b / 20b decode at
    # context 2048: 3.87 / 2.65 ms per token against 3.70 / 2.50 with one kernel per op: every CTA of the GEMV repeats the norm's
    # reads from L2, which costs more than the launch it saves under programmatic dependent launch.  Off; tests keep it honest.
    FUSED_DECODE = False
    FUSED_DECODE_QKV = True      # ... the attention norm inside the qkv GEMV
    FUSED_DECODE_ROUTER = True   # ... the FFN norm, routing and quantisation inside the router GEMV

    def _run_layers_decode(self, x, delta, fb, kv):
        """Single-rank decode (one or two rows): both norms of a layer run inside the GEMV that consumes them (qkv; router, whose launch
        also routes and quantises), so a layer is qkv -> head epilogue -> attention -> o-proj -> router -> gate|up -> down."""
        from ..ops import cuda as K_
        c, par = self.cfg, self.par
        nk = dict(one_plus_w=self.one_plus_w, delta_scale=c.residual_scale)
        for L in self.layers:
            at = L["attn"]
            r = None
            if self.FUSED_DECODE_QKV and isinstance(at.qkv, Linear):
                r = K_.gemv_norm(x, L["attn_norm"], c.rms_eps, at.qkv.w, at.qkv.bias, delta=delta, **nk)
            if r is None:
                qkv = at.qkv(self._norm(x, L["attn_norm"], delta))
            else:
                qkv, x, _ = r
            a = at.attend(qkv, fb, kv, self.rope, par)
            moe = L.get("moe")
            r = None
            if self.FUSED_DECODE_ROUTER and moe is not None and moe.mx is not None and moe.expert_scale is None and moe.shared is None:
                # with one token the down projection has too few (pair, column block) items for the chip: it splits K in two
                copies = K_.mxf4_ksplit(moe.mx[1].K, moe.DOWN_KSPLIT) if x.shape[0] * moe.K <= 4 else 1
                r = K_.gemv_norm(x, L["ffn_norm"], c.rms_eps, moe.router.w, moe.router.bias, delta=a, route=(moe.router_bias, moe.K, True, copies), **nk)
            if r is not None:
                _, x, _, idx, w, xq, sfx = r
                delta = moe(a, par, router_h=(idx, w, xq, sfx))        # (`a` only gives the row count here)
            else:
                h2 = self._norm(x, L["ffn_norm"], a)
                delta = moe(h2, par) if moe is not None else L["ffn"](h2, par)
        return x, delta

    def _run_layers(self, x, delta, fb, kv, state):
        par = self.par
        if (self.FUSED_DECODE and x.is_cuda and x.shape[0] <= 2 and par.world == 1 and self.tap is None and state is None
                and type(self) is TransformerModel and ops.backend() != "torch"):
            return self._run_layers_decode(x, delta, fb, kv)
        for li, L in enumerate(self.layers):
            h = self._norm(x, L["attn_norm"], delta)
            a = self._mixer(li, L, h, fb, kv, state)
            h2 = self._norm(x, L["ffn_norm"], a)
            delta = L["moe"](h2, par) if "moe" in L else L["ffn"](h2, par)
            if self.tap is not None:                 # per-layer dump hook of the parity tools (single rank, eager)
                if not isinstance(delta, torch.Tensor) and hasattr(delta, "materialize"):
                    delta = delta.materialize()
                self.tap(li, a, delta, x)
        return x, delta

    def _head(self, x, delta, fb):
        c, par = self.cfg, self.par
        rs = c.residual_scale
        rows = fb.logit_rows if fb.logit_rows is not None else (fb.cu_q[1:].long() - 1)
        xr = x.index_select(0, rows)
        dr = delta.index_select(0, rows).contiguous() if delta is not None else None       # (a pending fused reduction is summed here)
        hidden = None
        if fb.want_hidden:
            hidden = xr + dr.to(torch.float32) * rs if dr is not None else xr.clone()
        hn = ops.rmsnorm(xr, self.out_norm, c.rms_eps, delta=dr, one_plus_w=self.one_plus_w, delta_scale=rs)
        logits = self.lm_head(hn, out_f32=True)
        if self.vocab_hi - self.vocab_lo != c.vocab:
            logits = par.all_gather_cols(logits)
        if c.logit_scale != 1.0:
            logits = logits * c.logit_scale
        if c.final_logit_softcap > 0:
            logits = torch.tanh(logits / c.final_logit_softcap) * c.final_logit_softcap
        return (logits, hidden) if fb.want_hidden else logits

    # ---- layer-split (pipeline) forward
    def _forward_pipeline(self, fb: ForwardBatch, kv: KVCache, state=None):
        """Each rank runs its contiguous layer range.  A single long prefill chunk is cut into token micro-batches that
        flow through the stages back to back (stage r works on micro-batch i while stage r+1 works on i-1; causal
        attention only needs the earlier micro-batches' KV, which that stage has already written), so the stages
        overlap instead of running strictly one after the other as in the reference (src/model/dense_split.cpp:258:
        one residual hand-off per boundary, serial).  The residual crosses a boundary as one fp32 [T, H] message over
        NCCL point-to-point; the last stage's logits are broadcast so that every rank samples the same token."""
        c, par = self.cfg, self.par
        if fb.want_hidden:
            raise NotImplementedError("speculative decoding is not combined with the layer split")
        rows = fb.logit_rows if fb.logit_rows is not None else (fb.cu_q[1:].long() - 1)
        n_rows = rows.numel()
        out = None
        pieces = self._micro_batches(fb)
        last_logits = []
        for mb, keep in pieces:
            if self.first_stage:
                x = ops.embed(self.embed_w, mb.ids, c.embedding_scale)
            else:
                x = torch.empty(mb.T, c.hidden, dtype=torch.float32, device=self.device)
                par.recv(x, par.rank - 1)
            x, delta = self._run_layers(x, None, mb, kv, state)
            if not self.last_stage:
                d = delta if isinstance(delta, torch.Tensor) else delta.materialize()
                x = x + d.to(torch.float32) * c.residual_scale
                par.send(x.contiguous(), par.rank + 1)
            elif keep:
                last_logits.append(self._head(x, delta, mb))
        logits = torch.empty(n_rows, c.vocab, dtype=torch.float32, device=self.device)
        if self.last_stage:
            logits.copy_(torch.cat(last_logits, dim=0) if len(last_logits) > 1 else last_logits[0])
        par.broadcast(logits, src=par.world - 1)
        return logits

    def _micro_batches(self, fb: ForwardBatch, min_tokens: int = 256):
        """[(ForwardBatch, has_logit_rows)].  Only a single-sequence prefill chunk is cut (into world-size pieces of at
        least ``min_tokens``); mixed batches and decode steps go through whole."""
        n = self.par.world
        if fb.B != 1 or fb.T < 2 * min_tokens or fb.logit_rows is None or fb.state_slots is not None:
            return [(fb, True)]
        T = fb.T
        per = max(min_tokens, (T + n - 1) // n)
        per = (per + 127) // 128 * 128
        kv_end = int(fb.seq_lens[0])
        start = kv_end - T
        out, rows = [], fb.logit_rows
        for lo in range(0, T, per):
            hi = min(T, lo + per)
            sel = (rows >= lo) & (rows < hi)
            lr = (rows[sel] - lo)
            mb = ForwardBatch(fb.ids[lo:hi], fb.positions[lo:hi], fb.slot_map[lo:hi], fb.block_table,
                              torch.tensor([start + hi], dtype=torch.int32, device=fb.ids.device),
                              torch.tensor([0, hi - lo], dtype=torch.int32, device=fb.ids.device), hi - lo, logit_rows=lr if lr.numel() else None)
            out.append((mb, lr.numel() > 0))
        return out

    def _norm(self, x, w, delta):
        """Residual add + RMSNorm; a delta that still lives as per-rank partials in the collective inbox is summed here."""
        c = self.cfg
        if delta is not None and not isinstance(delta, torch.Tensor):
            if hasattr(delta, "pair_to_packed"):       # an expert combine that has not been formed (ops.cuda.CombineDelta)
                from ..ops.cuda import rmsnorm_combine
                return rmsnorm_combine(x, w, c.rms_eps, delta, one_plus_w=self.one_plus_w, delta_scale=c.residual_scale)
            return self.par.fused.rmsnorm(x, w, c.rms_eps, delta, one_plus_w=self.one_plus_w, delta_scale=c.residual_scale)
        return ops.rmsnorm(x, w, c.rms_eps, delta=delta, one_plus_w=self.one_plus_w, delta_scale=c.residual_scale)

    def _mixer(self, li, L, h, fb, kv, state):
        return L["attn"](h, fb, kv, self.rope, self.par)


def _bytes_of(v) -> int:
    if isinstance(v, torch.Tensor):
        return v.numel() * v.element_size()
    if isinstance(v, QuantWeight):
        return v.nbytes
    if isinstance(v, Linear):
        return v.w.nbytes + (_bytes_of(v.bias) if v.bias is not None else 0)
    if isinstance(v, MultiLinear):
        return sum(_bytes_of(p) for p in v.parts)
    if isinstance(v, (list, tuple)):
        return sum(_bytes_of(i) for i in v)
    if hasattr(v, "__dict__"):
        return sum(_bytes_of(i) for i in vars(v).values() if isinstance(i, (torch.Tensor, QuantWeight, Linear, MultiLinear, tuple, list)))
    return 0
