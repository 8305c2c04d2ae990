"""Gemma-4 (``gemma4``): per-layer head geometry, sandwich norms, GeGLU, dense + routed dual-path FFN, logit soft-cap.

Layer (reference parity: src/model/gemma4.cpp:648-985, include/ie/model_config.hpp:212-254):

    h   = rms(x, attn_norm)
    q,k = per-head rms(q_proj h, q_norm), rms(k_proj h, k_norm);  v = weightless per-head rms(v_proj h, or of the raw k projection
          on layers without attn_v);  partial NEOX RoPE with the layer's own dimension count and base (global layers may carry
          frequency factors);  attention with scale 1 (sliding window on the layers the pattern marks)
    a   = x + rms(o_proj attn, post_attention_norm)
    y   = down(gelu_tanh(gate rms(a, ffn_norm)) * up rms(a, ffn_norm))                       dense path, every layer
    MoE layers:  y = rms(y, post_ffw_norm_1) + rms(experts(rms(a, pre_ffw_norm_2)), post_ffw_norm_2)
                 router input = weightless rms(a) * ffn_gate_inp.scale / sqrt(H);  softmax over all experts, top-k, renormalised;
                 each expert's output is multiplied by ffn_down_exps.scale[e]
    x   = (a + rms(y, post_ffw_norm)) * layer_output_scale

Embeddings are scaled by sqrt(H); the tied head's logits pass through tanh soft-capping.  Sliding and global layers have
different head_dim and KV-head counts, so the paged cache keeps one tensor shape per layer.  The graph runs on one GPU (as
the reference's does); the assistant (MTP) head of the reference is not part of this class.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..formats.model_config import ModelConfig
from ..ops import ACT_GEGLU
from ..parallel.comm import ParallelCtx
from ..utils.rope import rope_tables
from .transformer import AttentionBlock, DenseFFN, ForwardBatch, KVCache, MoEFFN, TransformerModel


class Gemma4Model(TransformerModel):
    def __init__(self, cfg: ModelConfig, src, device, par: Optional[ParallelCtx] = None, max_ctx: int = 8192):
        par = par or ParallelCtx()
        if par.world > 1 and par.mode == "tp":
            raise ValueError("the Gemma-4 graph runs on one GPU (tensor parallelism is not wired for its per-layer head geometry)")
        self._ropes: dict = {}
        self._zero: Optional[torch.Tensor] = None
        self._acc: Optional[torch.Tensor] = None
        super().__init__(cfg, src, device, par, max_ctx=max_ctx)
        self.n_kv_local = max(int(v) for v in cfg.layer_n_kv)          # upper bounds, used to size the block pool
        self.kv_geometry = {l: (L["attn"].n_kv, L["attn"].hd) for l, L in zip(self.layer_ids, self.layers)}

    # ---- construction
    def _rope_for(self, layer: int, src):
        c = self.cfg
        _, _, n_rot, theta = c.layer_geometry(layer)
        swa = bool(c.layer_swa[layer])
        if swa not in self._ropes:
            ff = None
            if not swa and getattr(src, "r", None) is not None and src.has("rope_freqs.weight"):
                ff = src.vector("rope_freqs.weight", n_rot // 2)
            self._ropes[swa] = rope_tables(self.max_ctx, n_rot, theta, ff, device=self.device)
        return self._ropes[swa]

    def _build_layer(self, l: int, src) -> dict:
        c, par = self.cfg, self.par
        p, H = f"blk.{l}", c.hidden
        L = {"attn_norm": src.vector(f"{p}.attn_norm.weight", H), "attn": AttentionBlock(c, l, src, par), "rope": self._rope_for(l, src),
             "post_attn_norm": src.vector(f"{p}.post_attention_norm.weight", H), "ffn_norm": src.vector(f"{p}.ffn_norm.weight", H),
             "ffn": DenseFFN(c, l, src, par, act=ACT_GEGLU), "post_ffw_norm": src.vector(f"{p}.post_ffw_norm.weight", H)}
        from_file = getattr(src, "r", None) is not None
        L["out_scale"] = 1.0
        if not from_file or src.has(f"{p}.layer_output_scale.weight"):
            L["out_scale"] = float(src.vector(f"{p}.layer_output_scale.weight", 1)[0])
        if c.is_moe and (not from_file or src.has(f"{p}.ffn_gate_inp.weight")):
            moe = MoEFFN(c, l, src, par, ACT_GEGLU, with_bias=False)
            if not from_file or src.has(f"{p}.ffn_down_exps.scale"):
                moe.expert_scale = src.vector(f"{p}.ffn_down_exps.scale", c.n_experts).contiguous()
            rs = src.vector(f"{p}.ffn_gate_inp.scale", H) if (not from_file or src.has(f"{p}.ffn_gate_inp.scale")) else torch.ones(H, device=self.device)
            L.update(moe=moe, router_norm=(rs / math.sqrt(H)).contiguous(), pre_ffw_norm_2=src.vector(f"{p}.pre_ffw_norm_2.weight", H),
                     post_ffw_norm_1=src.vector(f"{p}.post_ffw_norm_1.weight", H), post_ffw_norm_2=src.vector(f"{p}.post_ffw_norm_2.weight", H))
        return L

    def new_kv_cache(self, num_blocks: int, dtype: str = "bf16") -> KVCache:
        return KVCache(self.cfg.n_layers, num_blocks, self.n_kv_local, self.cfg.head_dim, self.device, self.attn_layers, dtype=dtype,
                       geometry=self.kv_geometry)

    # ---- forward
    def _buffers(self, T: int):
        """(zeros, accumulator) fp32 [T, H].  Under graph capture they come from the graph's pool: a captured kernel keeps the raw
        address, and the shared pair below is re-allocated when a longer batch arrives."""
        H = self.cfg.hidden
        if self.device.type == "cuda" and torch.cuda.is_current_stream_capturing():
            return torch.zeros(T, H, dtype=torch.float32, device=self.device), torch.empty(T, H, dtype=torch.float32, device=self.device)
        if self._zero is None or self._zero.shape[0] < T:
            n = max(T, 256)
            self._zero = torch.zeros(n, H, dtype=torch.float32, device=self.device)
            self._acc = torch.zeros(n, H, dtype=torch.float32, device=self.device)
        return self._zero[:T], self._acc[:T]

    def _plain_norm(self, y: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """rms(y) * w of a tensor that is not the residual stream (bf16 or fp32 [T, H]) -> bf16."""
        zero, _ = self._buffers(y.shape[0])
        return ops.rmsnorm(zero, w, self.cfg.rms_eps, delta=y.contiguous(), write_x=False)

    def _run_layers(self, x, delta, fb: ForwardBatch, kv: KVCache, state):
        c, par, eps = self.cfg, self.par, self.cfg.rms_eps
        for li, L in enumerate(self.layers):
            h = ops.rmsnorm(x, L["attn_norm"], eps, delta=delta)
            o = self._plain_norm(L["attn"](h, fb, kv, L["rope"], par), L["post_attn_norm"])
            h2 = ops.rmsnorm(x, L["ffn_norm"], eps, delta=o)                 # x is now x + post_norm(attention)
            y = L["ffn"](h2, par)
            if "moe" in L:
                y1 = self._plain_norm(y, L["post_ffw_norm_1"])
                e_in = ops.rmsnorm(x, L["pre_ffw_norm_2"], eps)
                r_in = ops.rmsnorm(x, L["router_norm"], eps)
                m = self._plain_norm(L["moe"](e_in, par, router_h=r_in), L["post_ffw_norm_2"])
                _, acc = self._buffers(x.shape[0])
                acc.zero_()
                ops.scaled_add(acc, y1)
                y = ops.rmsnorm(acc, L["post_ffw_norm"], eps, delta=m, write_x=False)
            else:
                y = self._plain_norm(y, L["post_ffw_norm"])
            if self.tap is not None:
                self.tap(li, o, y, x)
            if L["out_scale"] != 1.0:
                ops.scaled_add(x, y)
                x.mul_(L["out_scale"])
                delta = None
            else:
                delta = y
        return x, delta
