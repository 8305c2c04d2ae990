"""Gemma-4 assistant head (``gemma4-assistant``): a small EAGLE-style draft model for greedy self-speculative decoding.

The head embeds the pending token with the TARGET's embedding table, concatenates the target's hidden state of the last committed
position, projects the pair down to its own width and runs a few sandwich-norm layers whose attention has queries only: keys and
values are the target's own cache, read in place (sliding-window head layers read the target's last sliding-window layer, global
head layers its last global layer -- layers n-2 and n-1 of the released checkpoints), so the head writes no cache and needs no
rollback.  It returns draft logits through its own (tied) token table and a recurrence hidden of the target's width that feeds the
next draft step.  All K drafts of a round are made at the same position p, the number of committed keys.

    x    = pre_projection([embed_target(tok) * sqrt(BB) ; h])                         BB = target hidden, H = head hidden
    per layer:  q = rope(per-head rms(Wq rms(x, attn_norm), q_norm));  a = attention(q, target K/V[0, p), scale 1)
                x1 = x + rms(Wo a, post_attention_norm);  y = down(gelu(gate rms(x1, ffn_norm)) * up(...))
                x  = (x1 + rms(y, post_ffw_norm)) * layer_output_scale
    logits = token_embd_head(rms(x, output_norm));   h_next = post_projection(rms(x, output_norm))

Reference parity: include/ie/gemma4_assistant.hpp:1-88, src/model/gemma4_assistant.cpp:10-153 (config keys and tensors),
src/model/gemma4.cpp:1053-1260 (load, one draft step, draft / verify loop), src/engine/engine.cpp:554-625 (engine wiring).
The verify loop is the engine's own (``runtime/engine.py``: one target forward over [pending, drafts], longest agreeing prefix).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field, replace
from typing import Optional

import torch

from .. import ops
from ..ops import ACT_GEGLU
from ..utils.rope import rope_tables
from .transformer import DenseFFN, Linear


@dataclass
class AssistantConfig:
    n_layers: int
    hidden: int                  # head width
    backbone: int                # target hidden (width of h and of the target's embedding rows)
    ffn: int
    vocab: int
    n_q_heads: int
    rms_eps: float = 1e-6
    sliding_window: int = 1024
    is_swa: list = field(default_factory=list)
    n_kv_heads: list = field(default_factory=list)
    head_dim: list = field(default_factory=list)
    n_rot: list = field(default_factory=list)
    rope_theta: list = field(default_factory=list)


def read_assistant_config(kv: dict, tensors: dict) -> AssistantConfig:
    """``gemma4-assistant.*`` metadata of a head file; the backbone width comes from the post-projection's shape."""
    k = lambda s: f"gemma4-assistant.{s}"

    def need(s):
        if k(s) not in kv:
            raise ValueError(f"assistant head: missing {k(s)}")
        return kv[k(s)]

    L = int(need("block_count"))
    hd_g, hd_s = int(kv.get(k("attention.key_length"), 512)), int(kv.get(k("attention.key_length_swa"), 256))
    nr_g, nr_s = int(kv.get(k("rope.dimension_count"), hd_g)), int(kv.get(k("rope.dimension_count_swa"), hd_s))
    th_g, th_s = float(kv.get(k("rope.freq_base"), 1e6)), float(kv.get(k("rope.freq_base_swa"), 1e4))
    pat = kv.get(k("attention.sliding_window_pattern"))
    is_swa = [bool(v) for v in pat] if isinstance(pat, (list, tuple)) and len(pat) == L else [i + 1 != L for i in range(L)]
    nkv = need("attention.head_count_kv")
    n_kv = [int(v) for v in nkv] if isinstance(nkv, (list, tuple)) else [int(nkv)] * L
    if "token_embd.weight" not in tensors or "nextn.post_projection.weight" not in tensors:
        raise ValueError("assistant head: token_embd.weight / nextn.post_projection.weight missing")
    vocab = int(tensors["token_embd.weight"].shape[0])
    backbone = int(tensors["nextn.post_projection.weight"].shape[0])
    return AssistantConfig(L, int(need("embedding_length")), backbone, int(need("feed_forward_length")), vocab, int(need("attention.head_count")),
                           float(kv.get(k("attention.layer_norm_rms_epsilon"), 1e-6)), int(kv.get(k("attention.sliding_window"), 1024)),
                           is_swa, n_kv, [hd_s if s else hd_g for s in is_swa], [nr_s if s else nr_g for s in is_swa],
                           [th_s if s else th_g for s in is_swa])


def synth_assistant_config(target, n_layers: int = 2, hidden: int = 0, ffn: int = 0) -> AssistantConfig:
    """A head that fits a target configuration (random-init graphs and tests): sliding-window layers, then one global layer, each with
    the geometry of the target layer whose cache it reads."""
    c = target
    hidden = hidden or max(64, c.hidden // 2)
    is_swa = [i + 1 != n_layers for i in range(n_layers)]
    geo = {s: c.layer_geometry(_shared_layer(c, s)) for s in set(is_swa)}
    return AssistantConfig(n_layers, hidden, c.hidden, ffn or 2 * hidden, c.vocab, c.n_heads, c.rms_eps, c.sliding_window or 1024, is_swa,
                           [geo[s][1] for s in is_swa], [geo[s][0] for s in is_swa], [geo[s][2] for s in is_swa], [geo[s][3] for s in is_swa])


def _shared_layer(target_cfg, swa: bool) -> int:
    """The target layer whose cache a head layer of this kind reads: the last sliding-window / the last global layer."""
    for l in range(target_cfg.n_layers - 1, -1, -1):
        if bool(target_cfg.layer_swa[l]) == swa:
            return l
    raise ValueError("the target has no " + ("sliding-window" if swa else "global") + " layer for the assistant head to share")


class Gemma4AssistantHead:
    def __init__(self, model, src, cfg: AssistantConfig):
        """``model``: the loaded Gemma-4 target; ``src``: weight source of the head (a GGUF source or a synthetic one)."""
        t = model.cfg
        if cfg.vocab != t.vocab:
            raise ValueError(f"assistant head: vocab {cfg.vocab} != target vocab {t.vocab}")
        if cfg.backbone != t.hidden:
            raise ValueError(f"assistant head: backbone width {cfg.backbone} != target hidden {t.hidden}")
        self.model, self.cfg = model, cfg
        dev = model.device
        H, BB = cfg.hidden, cfg.backbone
        self.pre = Linear(src.matrix("nextn.pre_projection.weight", H, 2 * BB))
        self.post = Linear(src.matrix("nextn.post_projection.weight", BB, H))
        self.tok = Linear(src.matrix("token_embd.weight", cfg.vocab, H))          # the head's own table: its logits
        self.out_norm = src.vector("output_norm.weight", H)
        from_file = getattr(src, "r", None) is not None
        ff = src.vector("rope_freqs.weight", max(cfg.n_rot) // 2) if (from_file and src.has("rope_freqs.weight")) else None
        ffn_cfg = replace(t, hidden=H, ffn=cfg.ffn)
        self.layers = []
        ropes: dict = {}
        for l in range(cfg.n_layers):
            p = f"blk.{l}"
            swa, hd, n_kv = bool(cfg.is_swa[l]), cfg.head_dim[l], cfg.n_kv_heads[l]
            shared = _shared_layer(t, swa)
            thd, tkv, _, _ = t.layer_geometry(shared)
            if (thd, tkv) != (hd, n_kv):
                raise ValueError(f"assistant head layer {l}: geometry ({hd}, {n_kv} kv heads) differs from target layer {shared} ({thd}, {tkv})")
            if swa not in ropes:
                ropes[swa] = rope_tables(model.max_ctx, cfg.n_rot[l], cfg.rope_theta[l], None if swa else ff, device=dev)
            scale = 1.0
            if not from_file or src.has(f"{p}.layer_output_scale.weight"):
                scale = float(src.vector(f"{p}.layer_output_scale.weight", 1)[0])
            self.layers.append(dict(
                swa=swa, hd=hd, n_rot=cfg.n_rot[l], shared=shared, rope=ropes[swa], out_scale=scale,
                attn_norm=src.vector(f"{p}.attn_norm.weight", H), q_norm=src.vector(f"{p}.attn_q_norm.weight", hd),
                post_attn_norm=src.vector(f"{p}.post_attention_norm.weight", H), ffn_norm=src.vector(f"{p}.ffn_norm.weight", H),
                post_ffw_norm=src.vector(f"{p}.post_ffw_norm.weight", H),
                wq=Linear(src.matrix(f"{p}.attn_q.weight", cfg.n_q_heads * hd, H)), wo=Linear(src.matrix(f"{p}.attn_output.weight", H, cfg.n_q_heads * hd)),
                ffn=DenseFFN(ffn_cfg, l, src, model.par, act=ACT_GEGLU)))
        self._zero = torch.zeros(1, max(H, BB), dtype=torch.float32, device=dev)
        self._cu = torch.tensor([0, 1], dtype=torch.int32, device=dev)
        self._noslot = torch.full((1,), -1, dtype=torch.int64, device=dev)

    def _plain_norm(self, y: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(self._zero[:, :y.shape[1]].contiguous(), w, self.cfg.rms_eps, delta=y.contiguous(), write_x=False)

    def step(self, h: torch.Tensor, tok: int, p: int, kv, block_table: torch.Tensor):
        """One draft step at position ``p`` (keys [0, p) of the target cache are read).  ``h`` fp32 [1, BB].  Returns
        (logits fp32 [1, vocab], h_next fp32 [1, BB])."""
        m, c, t = self.model, self.cfg, self.model.cfg
        dev = m.device
        ids = torch.tensor([tok], dtype=torch.int32, device=dev)
        e = ops.embed(m.embed_w, ids, math.sqrt(c.backbone))
        xin = torch.cat([e.to(torch.bfloat16), h.to(torch.bfloat16)], dim=1).contiguous()
        x = self.pre(xin, out_f32=True)
        pos = torch.tensor([p], dtype=torch.int32, device=dev)
        seq = torch.tensor([p], dtype=torch.int32, device=dev)
        delta = None
        for L in self.layers:
            xn = ops.rmsnorm(x, L["attn_norm"], c.rms_eps, delta=delta)
            k_c, v_c = kv.k[L["shared"]], kv.v[L["shared"]]
            q, _ = ops.qkv_post(L["wq"](xn), None, L["q_norm"], None, pos, L["rope"][0], L["rope"][1], self._noslot, k_c, v_c, c.n_q_heads, 0,
                                L["hd"], L["n_rot"], eps=c.rms_eps, kv_scales=kv.scales(L["shared"]))
            a = ops.attention(q, k_c, v_c, block_table, seq, self._cu, 1, window=c.sliding_window if L["swa"] else 0, scale=1.0,
                              kv_scales=kv.scales(L["shared"]), max_kv_len=p)
            o = self._plain_norm(L["wo"](a.reshape(1, -1)), L["post_attn_norm"])
            xn = ops.rmsnorm(x, L["ffn_norm"], c.rms_eps, delta=o)                    # x is now x + rms(o_proj attention)
            y = self._plain_norm(L["ffn"](xn, m.par), L["post_ffw_norm"])
            if L["out_scale"] != 1.0:
                ops.scaled_add(x, y)
                x.mul_(L["out_scale"])
                delta = None
            else:
                delta = y
        xn = ops.rmsnorm(x, self.out_norm, c.rms_eps, delta=delta)
        return self.tok(xn, out_f32=True), self.post(xn, out_f32=True)

    def draft(self, h_last: torch.Tensor, tok: int, k: int, ctx: Optional[dict] = None) -> list:
        """Greedy draft of ``k`` tokens after the pending token ``tok``.  ``ctx``: the engine's view of the sequence -- ``kv`` (the
        target's cache), ``block_table`` (int32 [1, blocks]) and ``pos`` (committed keys)."""
        if ctx is None:
            raise ValueError("the Gemma-4 assistant head reads the target's KV cache: draft() needs the sequence context")
        out, h = [], h_last
        for _ in range(k):
            logits, h = self.step(h, tok, int(ctx["pos"]), ctx["kv"], ctx["block_table"])
            tok = int(ops.argmax(logits)[0])
            out.append(tok)
        return out


def load_assistant_head(model, path: str):
    """Opens a ``gemma4-assistant`` GGUF and attaches the head to the loaded target as ``model.mtp``."""
    from ..formats.gguf import GGUFReader
    from .sources import GGUFSource
    reader = GGUFReader(path)
    arch = reader.kv.get("general.architecture")
    if arch != "gemma4-assistant":
        raise ValueError(f"{path}: general.architecture is {arch!r}, expected 'gemma4-assistant'")
    if model.cfg.arch != "gemma4":
        raise ValueError("the gemma4-assistant head drafts for a Gemma-4 target only")
    cfg = read_assistant_config(reader.kv, reader.tensors)
    model.mtp = Gemma4AssistantHead(model, GGUFSource(reader, model.device), cfg)
    return model.mtp


def attach_synth_head(model, quant: str = "q8_0", seed: int = 7, **kw):
    """Random-init head for a random-init target (tests, benchmarks without a checkpoint)."""
    from .sources import SynthSource, default_policy
    cfg = synth_assistant_config(model.cfg, **kw)
    src = SynthSource(model.device, default_policy("gemma4", quant), seed=seed, n_layers=cfg.n_layers, gen_device="cpu")
    model.mtp = Gemma4AssistantHead(model, src, cfg)
    return model.mtp
