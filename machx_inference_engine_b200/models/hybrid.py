"""Hybrid graphs: gated-DeltaNet (linear attention) layers interleaved with gated full-attention layers.

Families: Qwen3-Next-80B-A3B (``qwen3next``: 3 DeltaNet + 1 attention per group, 512-expert MoE + sigmoid-gated
shared expert), Qwen3.6-35B-A3B (``qwen35moe``) and Qwen3.6-27B (``qwen35``, dense SwiGLU FFN).  Reference parity:
src/model/qwen3next.cpp:620-1064 (layer bodies), src/model/qwen36.cpp, src/model/qwen35_dense.cpp (tile repeat,
separate alpha/beta projections, MTP head :1000-1264).  One class serves the three families and every parallel form;
the reference keeps a copy of the forward per family and per split/TP variant.

DeltaNet layer:  x -> [qkv | z | beta,alpha] projection (one GEMM) -> causal conv1d+SiLU over the qkv channels
-> gated delta-rule scan (L2-norm, g/beta and head repeat fused in the kernel) -> gated RMSNorm with z -> out proj.
Tensor parallelism shards k/v heads (and the conv channels with them); recurrent state and conv state are per rank.

The MTP head drafts tokens for greedy self-speculative decoding; the verify forward runs in checkpoint mode (state
snapshots after every position) so a partially accepted draft rolls the recurrent state back without recomputation.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..formats.model_config import ModelConfig
from ..ops import ACT_SWIGLU, QuantWeight
from ..parallel.comm import ParallelCtx
from .transformer import AttentionBlock, DenseFFN, ForwardBatch, KVCache, Linear, MoEFFN, TransformerModel, _fuse_rows

D_HEAD = 128      # DeltaNet key / value head width (the only geometry the families use)


class DeltaNetState:
    """Recurrent state of every DeltaNet layer for ``n_slots`` concurrent sequences (include/ie/deltanet_state.hpp:28-75):
    ``S[l]`` fp32 [slots, n_v, 128 (v), 128 (k)] and ``conv[l]`` bf16 [slots, kernel-1, channels]."""

    def __init__(self, layers: list, n_slots: int, n_v: int, channels: int, kernel: int, device):
        self.layers, self.n_slots, self.n_v, self.channels, self.kernel, self.device = layers, n_slots, n_v, channels, kernel, device
        self.S = {l: torch.zeros(n_slots, n_v, D_HEAD, D_HEAD, dtype=torch.float32, device=device) for l in layers}
        self.conv = {l: torch.zeros(n_slots, kernel - 1, channels, dtype=torch.bfloat16, device=device) for l in layers}
        self.ckpt_S: dict = {}
        self.ckpt_conv: dict = {}
        self.ckpt_rows = 0

    def reset(self, slots) -> None:
        idx = torch.as_tensor(list(slots), dtype=torch.long, device=self.device)
        if idx.numel() == 0:
            return
        for l in self.layers:
            self.S[l].index_fill_(0, idx, 0.0)
            self.conv[l].index_fill_(0, idx, 0.0)

    def copy_slot(self, src: int, dst: int) -> None:
        for l in self.layers:
            self.S[l][dst].copy_(self.S[l][src])
            self.conv[l][dst].copy_(self.conv[l][src])

    def snapshot(self, slot: int) -> dict:
        return {"S": {l: self.S[l][slot].clone() for l in self.layers}, "conv": {l: self.conv[l][slot].clone() for l in self.layers}}

    def restore(self, slot: int, snap: dict) -> None:
        for l in self.layers:
            self.S[l][slot].copy_(snap["S"][l])
            self.conv[l][slot].copy_(snap["conv"][l])

    # ---- per-position checkpoints of one verify step (Qwen35SpecCheckpoint, src/model/qwen35_dense.cpp:892-937)
    def enable_checkpoints(self, rows: int) -> None:
        if rows > self.ckpt_rows:
            self.ckpt_S = {l: torch.empty(rows, self.n_v, D_HEAD, D_HEAD, dtype=torch.float32, device=self.device) for l in self.layers}
            self.ckpt_conv = {l: torch.empty(rows, self.kernel - 1, self.channels, dtype=torch.bfloat16, device=self.device) for l in self.layers}
            self.ckpt_rows = rows

    def commit(self, slot: int, row: int) -> None:
        """state[slot] <- the checkpoint taken after token row ``row`` of the last checkpointed forward."""
        for l in self.layers:
            self.S[l][slot].copy_(self.ckpt_S[l][row])
            self.conv[l][slot].copy_(self.ckpt_conv[l][row])

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for d in (self.S, self.conv) for t in d.values())


class LinearAttentionBlock:
    def __init__(self, cfg: ModelConfig, layer: int, src, par: ParallelCtx):
        c, p = cfg, f"blk.{layer}"
        H, n_k, n_v, Kc = c.hidden, c.ssm_n_k_heads, c.ssm_n_v_heads, c.ssm_conv_kernel
        if c.ssm_state != D_HEAD or c.ssm_inner != n_v * D_HEAD or n_v % n_k:
            raise ValueError("DeltaNet geometry must be 128-wide heads with n_v a multiple of n_k")
        rep = n_v // n_k
        tp = par.world if par.mode == "tp" else 1
        self.sharded = tp > 1 and n_k % tp == 0
        interleave = c.arch == "qwen3next"        # k-head h feeds v-heads rep*h .. rep*h+rep-1; the Qwen3.6 files tile instead
        kh = list(range(par.rank * (n_k // tp), (par.rank + 1) * (n_k // tp))) if self.sharded else list(range(n_k))
        vh = [k * rep + r for k in kh for r in range(rep)] if interleave else [k + j * n_k for j in range(rep) for k in kh]
        if not interleave:
            vh.sort()
        self.layer, self.n_k, self.n_v, self.Kc = layer, len(kh), len(vh), Kc
        self.C = (2 * self.n_k + self.n_v) * D_HEAD
        self.eps = c.rms_eps
        dev = None

        def rows_of(heads, base):
            return torch.cat([torch.arange(h * D_HEAD, (h + 1) * D_HEAD) for h in heads]) + base

        conv_rows = torch.cat([rows_of(kh, 0), rows_of(kh, n_k * D_HEAD), rows_of(vh, 2 * n_k * D_HEAD)])
        full_C = (2 * n_k + n_v) * D_HEAD
        w_qkv = src.matrix(f"{p}.attn_qkv.weight", full_C, H)
        w_z = src.matrix(f"{p}.attn_gate.weight", n_v * D_HEAD, H)
        if self.sharded:
            w_qkv, w_z = w_qkv.select_rows(conv_rows), w_z.select_rows(rows_of(vh, 0))
        parts, biases = [w_qkv, w_z], [None, None]
        k_local = {k: i for i, k in enumerate(kh)}
        if src.has(f"{p}.ssm_ba.weight") and c.arch == "qwen3next":
            # fused projection, per k-head group [beta (rep) | alpha (rep)] (src/model/qwen3next.cpp:731-747)
            w_ba = src.matrix(f"{p}.ssm_ba.weight", 2 * n_v, H)
            if self.sharded:
                w_ba = w_ba.select_rows(torch.cat([torch.arange(k * 2 * rep, (k + 1) * 2 * rep) for k in kh]))
            parts.append(w_ba); biases.append(None)
            b_idx = [k_local[v // rep] * 2 * rep + v % rep for v in vh]
            a_idx = [i + rep for i in b_idx]
        else:
            w_a = src.matrix(f"{p}.ssm_alpha.weight", n_v, H)
            w_b = src.matrix(f"{p}.ssm_beta.weight", n_v, H)
            if self.sharded:
                sel = torch.tensor(vh)
                w_a, w_b = w_a.select_rows(sel), w_b.select_rows(sel)
            parts += [w_a, w_b]; biases += [None, None]
            a_idx = list(range(self.n_v))
            b_idx = [self.n_v + i for i in range(self.n_v)]
        self.proj = _fuse_rows(parts, biases)
        self.z_off = self.C
        self.ab_off = self.C + self.n_v * D_HEAD
        conv_w = src.table(f"{p}.ssm_conv1d.weight", (full_C, Kc))
        self.conv_w = (conv_w[conv_rows.to(conv_w.device)] if self.sharded else conv_w).to(torch.float32).contiguous()
        dev = self.conv_w.device
        sel_v = torch.tensor(vh, device=dev)
        self.ssm_a = src.vector(f"{p}.ssm_a", n_v)[sel_v].contiguous()
        self.dt_bias = src.vector(f"{p}.ssm_dt.bias", n_v)[sel_v].contiguous()
        self.norm_w = src.vector(f"{p}.ssm_norm.weight", D_HEAD)
        self.a_idx = torch.tensor(a_idx, dtype=torch.int32, device=dev)
        self.b_idx = torch.tensor(b_idx, dtype=torch.int32, device=dev)
        self.k_of_v = torch.tensor([k_local[(v // rep) if interleave else (v % n_k)] for v in vh], dtype=torch.int32, device=dev)
        w_out = src.matrix(f"{p}.ssm_out.weight", H, n_v * D_HEAD)
        if self.sharded:
            # v-heads of a rank are contiguous under the interleaved mapping; the tiled mapping gathers columns
            if interleave:
                w_out = w_out.slice_k(vh[0] * D_HEAD, (vh[-1] + 1) * D_HEAD, requant=True)
            else:
                d = w_out.dequantize(torch.bfloat16).reshape(H, n_v * D_HEAD)[:, rows_of(vh, 0).to(w_out.device)]
                w_out = QuantWeight(ops.WFormat.BF16, H, len(vh) * D_HEAD, 1, d.contiguous().unsqueeze(0))
        self.out = Linear(w_out, reduce=self.sharded)

    def __call__(self, h: torch.Tensor, fb: ForwardBatch, state: DeltaNetState, par: ParallelCtx, checkpoint: bool = False):
        y = self.proj(h)                                           # [T, C | n_v*128 | alpha/beta]
        l = self.layer
        conv = ops.conv1d_silu(y[:, :self.C], self.conv_w, state.conv[l], fb.state_slots, fb.cu_q, fb.max_q_len,
                               ckpt=state.ckpt_conv[l] if checkpoint else None)
        o = ops.deltanet_scan(conv, self.n_k, y[:, self.ab_off:], self.a_idx, self.b_idx, self.k_of_v, self.ssm_a, self.dt_bias,
                              state.S[l], fb.state_slots, fb.cu_q, self.n_v, eps=1e-6, ckpt=state.ckpt_S[l] if checkpoint else None)
        g = ops.gated_rmsnorm_heads(o, y[:, self.z_off:self.z_off + self.n_v * D_HEAD], self.norm_w, self.eps, D_HEAD)
        return self.out(g, par if self.sharded else None)


class SharedExpert:
    """Always-on expert whose output is scaled by sigmoid(w_gate . x) per token (src/model/qwen3next.cpp:1053-1064);
    returns this rank's fp32 partial, to be summed into the MoE partial before the single reduction."""

    def __init__(self, cfg: ModelConfig, layer: int, src, par: ParallelCtx, prefix: Optional[str] = None):
        p = prefix or f"blk.{layer}"
        self.ffn = DenseFFN(cfg, layer, src, par, prefix=p, ffn=cfg.shared_expert_ffn, suffix="_shexp")
        self.ffn.down.reduce = False
        g = src.vector(f"{p}.ffn_gate_inp_shexp.weight", cfg.hidden)
        self.gate = Linear(QuantWeight(ops.WFormat.BF16, 1, cfg.hidden, 1, g.to(torch.bfloat16).reshape(1, 1, -1).contiguous()))

    def add_into(self, out: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        y = self.ffn(h, None)
        logit = self.gate(h, out_f32=True).reshape(-1)
        return ops.scaled_add(out, y, logit)


class MtpHead:
    """Multi-token-prediction draft head stored as layer ``n_layers`` of the checkpoint:
    x = eh_proj([enorm(embed(tok)) ; hnorm(h_prev)]) -> one gated-attention block with a private KV window -> FFN
    -> shared_head_norm -> the model's lm_head (src/model/qwen35_dense.cpp:1037-1155)."""

    def __init__(self, model: "HybridModel", src):
        c, par = model.cfg, model.par
        self.model = model
        l = c.n_layers
        p = f"blk.{l}"
        H = c.hidden
        self.eh = Linear(src.matrix(f"{p}.nextn.eh_proj.weight", H, 2 * H))
        self.enorm = src.vector(f"{p}.nextn.enorm.weight", H)
        self.hnorm = src.vector(f"{p}.nextn.hnorm.weight", H)
        self.shead_norm = src.vector(f"{p}.nextn.shared_head_norm.weight", H)
        self.attn_norm = src.vector(f"{p}.attn_norm.weight", H)
        self.post_norm = src.vector(f"{p}.post_attention_norm.weight", H)
        self.attn = AttentionBlock(c, l, src, par, q_gate=True)
        if c.is_moe:
            self.ffn = MoEFFN(c, l, src, par, ACT_SWIGLU, with_bias=False)
            if c.shared_expert_ffn:
                self.ffn.shared = SharedExpert(c, l, src, par)
        else:
            self.ffn = DenseFFN(c, l, src, par)
        self.kv = KVCache(1, 1, self.attn.n_kv, c.head_dim, model.device, [l])      # one page: the draft window of a round
        dev = model.device
        self._bt = torch.zeros(1, 1, dtype=torch.int32, device=dev)
        self._cu = torch.tensor([0, 1], dtype=torch.int32, device=dev)

    def draft(self, h_last: torch.Tensor, tok: int, k: int, ctx=None) -> list:
        """Greedy draft of ``k`` tokens from the hidden state (fp32 [1, H], before the final norm) of the last
        committed position and the token sampled there.  (``ctx``, the engine's view of the sequence, is not needed: this head keeps
        its own one-page cache.)"""
        m, c = self.model, self.model.cfg
        dev = m.device
        out = []
        h_src = h_last
        for j in range(k):
            ids = torch.tensor([tok], dtype=torch.int32, device=dev)
            e = ops.embed(m.embed_w, ids, c.embedding_scale)
            en = ops.rmsnorm(e, self.enorm, c.rms_eps, one_plus_w=m.one_plus_w, write_x=False)
            hn = ops.rmsnorm(h_src.clone(), self.hnorm, c.rms_eps, one_plus_w=m.one_plus_w, write_x=False)
            x = self.eh(torch.cat([en, hn], dim=1).contiguous(), out_f32=True)
            fb = ForwardBatch(ids=ids, positions=torch.tensor([j], dtype=torch.int32, device=dev),
                              slot_map=torch.tensor([j], dtype=torch.int64, device=dev), block_table=self._bt,
                              seq_lens=torch.tensor([j + 1], dtype=torch.int32, device=dev), cu_q=self._cu, max_q_len=1)
            xn = ops.rmsnorm(x, self.attn_norm, c.rms_eps, one_plus_w=m.one_plus_w, write_x=False)
            a = self.attn(xn, fb, self.kv, m.rope, m.par)
            xn = m._norm(x, self.post_norm, a)
            f = self.ffn(xn, m.par)
            hn = m._norm(x, self.shead_norm, f)            # x now holds the block output (next round's h_prev)
            logits = m.lm_head(hn, out_f32=True)
            if m.vocab_hi - m.vocab_lo != c.vocab:
                logits = m.par.all_gather_cols(logits)
            tok = int(ops.argmax(logits)[0])
            out.append(tok)
            h_src = x
        return out


class HybridModel(TransformerModel):
    needs_state = True

    def __init__(self, cfg: ModelConfig, src, device, par: Optional[ParallelCtx] = None, max_ctx: int = 8192):
        super().__init__(cfg, src, device, par, max_ctx)
        self.one_plus_w = cfg.arch in ("qwen35", "qwen35moe")       # Qwen3-Next files already hold 1 + w
        self.lin_layers = [l for l in self.layer_ids if not cfg.layer_is_full_attention(l)]
        self.mtp = MtpHead(self, src) if (cfg.nextn_predict_layers > 0 and not self.pp and src.has(f"blk.{cfg.n_layers}.nextn.eh_proj.weight")) else None

    def _build_layer(self, l: int, src) -> dict:
        c, par = self.cfg, self.par
        p = f"blk.{l}"
        L = {"attn_norm": src.vector(f"{p}.attn_norm.weight", c.hidden)}
        if c.layer_is_full_attention(l):
            L["attn"] = AttentionBlock(c, l, src, par, q_gate=True)
        else:
            L["lin"] = LinearAttentionBlock(c, l, src, par)
        L["ffn_norm"] = src.vector(f"{p}.post_attention_norm.weight", c.hidden)
        if c.is_moe:
            L["moe"] = MoEFFN(c, l, src, par, ACT_SWIGLU, with_bias=False)
            if c.shared_expert_ffn:
                L["moe"].shared = SharedExpert(c, l, src, par)
        else:
            L["ffn"] = DenseFFN(c, l, src, par)
        return L

    def new_state(self, n_slots: int) -> DeltaNetState:
        lin = next(L["lin"] for L in self.layers if "lin" in L)
        return DeltaNetState(self.lin_layers, n_slots, lin.n_v, lin.C, lin.Kc, self.device)

    def forward(self, fb: ForwardBatch, kv: KVCache, state: Optional[DeltaNetState] = None, checkpoint: bool = False):
        if state is None:
            raise ValueError("hybrid models need a DeltaNetState")
        if fb.start_host is not None:
            fresh = [fb.state_slots_host[i] for i, s in enumerate(fb.start_host) if s == 0]
            if fresh:
                state.reset(fresh)
        if checkpoint:
            state.enable_checkpoints(fb.T)
        self._ckpt = checkpoint
        try:
            return super().forward(fb, kv, state)
        finally:
            self._ckpt = False

    def _mixer(self, li, L, h, fb, kv, state):
        if "attn" in L:
            return L["attn"](h, fb, kv, self.rope, self.par)
        return L["lin"](h, fb, state, self.par, checkpoint=getattr(self, "_ckpt", False))
