"""Synthetic checkpoints: writes a complete GGUF (metadata, byte-level BPE tokenizer, every tensor of the architecture)
with random-init weights of a named configuration, so that the whole file path -- loader, repack, tokenizer, chat
template, server -- can be exercised on a box without any real checkpoint.

Tensor names, shapes (ggml order: contiguous/input dimension first, experts last) and the quantisation recipes follow
what llama.cpp-converted files of each family contain (the naming the reference loads: src/model/dense_transformer.cpp,
gptoss.cpp:96-214, qwen3moe.cpp, qwen3next.cpp:125-330, qwen35_dense.cpp:1037-1040).  Payloads are produced one tensor
at a time by the streaming writer, so a multi-GB file never needs more than one tensor in memory.
"""
from __future__ import annotations

import zlib
from typing import Callable, Iterable

import numpy as np

from .gguf import GGMLType, GGUFWriter, block_elems
from .model_config import ModelConfig, config_to_kv
from .quant import quantize

_CHATML_TEMPLATE = "{% for m in messages %}<|im_start|>{{ m.role }}\n{{ m.content }}<|im_end|>\n{% endfor %}<|im_start|>assistant\n"
_LLAMA3_TEMPLATE = "{% for m in messages %}<|start_header_id|>{{ m.role }}<|end_header_id|>\n\n{{ m.content }}<|eot_id|>{% endfor %}"
_HARMONY_TEMPLATE = "{% for m in messages %}<|start|>{{ m.role }}<|channel|>final<|message|>{{ m.content }}<|end|>{% endfor %}"


def gpt2_byte_map() -> list:
    """byte value -> the printable unicode character GPT-2 style vocabularies use for it."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    m = dict(zip(bs, cs))
    return [chr(m[b]) for b in range(256)]


def synthetic_tokenizer_kv(cfg: ModelConfig) -> dict:
    """A byte-level BPE vocabulary of exactly ``cfg.vocab`` entries: 256 byte tokens, a few real merges, the
    special tokens of the family's chat template, then filler words."""
    bm = gpt2_byte_map()
    tokens = list(bm)
    types = [1] * 256
    enc = lambda s: "".join(bm[b] for b in s.encode())
    merges = []
    words = ["the", " the", " a", "in", " in", "er", " of", "and", " and", "ing", " to", "on", " is", "Hello", " world", "\n\n", "  "]
    have = set(tokens)
    for w in words:
        e = enc(w)
        parts = [e[0]]
        for ch in e[1:]:
            a, b = parts[-1], ch
            if a + b not in have and len(tokens) < cfg.vocab - 64:
                merges.append(f"{a} {b}")
                tokens.append(a + b)
                types.append(1)
                have.add(a + b)
            parts[-1] = a + b
    fam = "harmony" if cfg.arch == "gpt-oss" else ("llama3" if cfg.arch == "llama" else "chatml")
    specials = {
        "chatml": ["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<tool_call>", "</tool_call>", "<think>", "</think>"],
        "llama3": ["<|begin_of_text|>", "<|end_of_text|>", "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>", "<|eom_id|>"],
        "harmony": ["<|endoftext|>", "<|start|>", "<|end|>", "<|message|>", "<|channel|>", "<|return|>", "<|call|>", "<|constrain|>"],
    }[fam]
    n_fill = cfg.vocab - len(tokens) - len(specials)
    if n_fill < 0:
        raise ValueError(f"vocabulary of {cfg.vocab} is too small for the synthetic tokenizer")
    for i in range(n_fill):
        tokens.append(enc(f" w{i}"))
        types.append(1)
    first_special = len(tokens)
    tokens += specials
    types += [3] * len(specials)
    ids = {s: first_special + i for i, s in enumerate(specials)}
    kv = {
        "tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": "llama-bpe" if fam == "llama3" else ("gpt-4o" if fam == "harmony" else "qwen2"),
        "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.token_type": types, "tokenizer.ggml.merges": merges,
        "tokenizer.chat_template": {"chatml": _CHATML_TEMPLATE, "llama3": _LLAMA3_TEMPLATE, "harmony": _HARMONY_TEMPLATE}[fam],
    }
    if fam == "llama3":
        kv["tokenizer.ggml.bos_token_id"] = ids["<|begin_of_text|>"]
        kv["tokenizer.ggml.eos_token_id"] = ids["<|eot_id|>"]
    elif fam == "harmony":
        kv["tokenizer.ggml.eos_token_id"] = ids["<|return|>"]
        kv["tokenizer.ggml.padding_token_id"] = ids["<|endoftext|>"]
    else:
        kv["tokenizer.ggml.eos_token_id"] = ids["<|im_end|>"]
        kv["tokenizer.ggml.padding_token_id"] = ids["<|endoftext|>"]
        kv["tokenizer.ggml.add_bos_token"] = False
    return kv


def tensor_plan(c: ModelConfig) -> list:
    """[(name, kind, dims)] for every tensor of the architecture; ``kind`` in matrix | expert | router | router_sharp | norm | qnorm | vector | conv | ssm_a.
    ``dims`` are ggml-ordered."""
    H, hd = c.hidden, c.head_dim
    out = [("token_embd.weight", "matrix", (H, c.vocab)), ("output_norm.weight", "norm", (H,))]
    if c.arch == "gemma4":
        return out + _gemma4_plan(c)
    if not c.tie_embeddings:
        out.append(("output.weight", "matrix", (H, c.vocab)))
    q_gate = c.is_hybrid

    def attention(p):
        if c.arch == "phi3":         # Phi-3 files keep q, k and v rows in one fused matrix
            return [(f"{p}.attn_qkv.weight", "matrix", (H, (c.n_heads + 2 * c.n_kv_heads) * hd)), (f"{p}.attn_output.weight", "matrix", (c.n_heads * hd, H))]
        t = [(f"{p}.attn_q.weight", "matrix", (H, c.n_heads * hd * (2 if q_gate else 1))), (f"{p}.attn_k.weight", "matrix", (H, c.n_kv_heads * hd)),
             (f"{p}.attn_v.weight", "matrix", (H, c.n_kv_heads * hd)), (f"{p}.attn_output.weight", "matrix", (c.n_heads * hd, H))]
        if c.arch in ("qwen2", "gpt-oss"):
            t += [(f"{p}.attn_q.bias", "vector", (c.n_heads * hd,)), (f"{p}.attn_k.bias", "vector", (c.n_kv_heads * hd,)),
                  (f"{p}.attn_v.bias", "vector", (c.n_kv_heads * hd,))]
        if c.arch == "gpt-oss":
            t += [(f"{p}.attn_output.bias", "vector", (H,)), (f"{p}.attn_sinks.weight", "vector", (c.n_heads,))]
        if c.arch in ("qwen3", "qwen3moe", "qwen3next", "qwen35", "qwen35moe"):
            t += [(f"{p}.attn_q_norm.weight", "norm", (hd,)), (f"{p}.attn_k_norm.weight", "norm", (hd,))]
        return t

    def linear_attention(p):
        n_k, n_v, D = c.ssm_n_k_heads, c.ssm_n_v_heads, c.ssm_state
        C = (2 * n_k + n_v) * D
        t = [(f"{p}.attn_qkv.weight", "matrix", (H, C)), (f"{p}.attn_gate.weight", "matrix", (H, n_v * D)),
             (f"{p}.ssm_conv1d.weight", "conv", (c.ssm_conv_kernel, C)), (f"{p}.ssm_a", "ssm_a", (n_v,)), (f"{p}.ssm_dt.bias", "vector", (n_v,)),
             (f"{p}.ssm_norm.weight", "norm", (D,)), (f"{p}.ssm_out.weight", "matrix", (n_v * D, H))]
        if c.arch == "qwen3next":
            t.append((f"{p}.ssm_ba.weight", "matrix", (H, 2 * n_v)))
        else:
            t += [(f"{p}.ssm_alpha.weight", "matrix", (H, n_v)), (f"{p}.ssm_beta.weight", "matrix", (H, n_v))]
        return t

    def ffn(p):
        if c.is_moe:
            E, F = c.n_experts, c.expert_ffn
            t = [(f"{p}.ffn_gate_inp.weight", "router", (H, E)), (f"{p}.ffn_gate_exps.weight", "expert", (H, F, E)),
                 (f"{p}.ffn_up_exps.weight", "expert", (H, F, E)), (f"{p}.ffn_down_exps.weight", "expert", (F, H, E))]
            if c.arch == "gpt-oss":
                t += [(f"{p}.ffn_gate_inp.bias", "vector", (E,)), (f"{p}.ffn_gate_exps.bias", "vector", (F, E)),
                      (f"{p}.ffn_up_exps.bias", "vector", (F, E)), (f"{p}.ffn_down_exps.bias", "vector", (H, E))]
            if c.shared_expert_ffn:
                S = c.shared_expert_ffn
                t += [(f"{p}.ffn_gate_inp_shexp.weight", "vector", (H,)), (f"{p}.ffn_gate_shexp.weight", "matrix", (H, S)),
                      (f"{p}.ffn_up_shexp.weight", "matrix", (H, S)), (f"{p}.ffn_down_shexp.weight", "matrix", (S, H))]
            return t
        if c.arch == "phi3":         # ... and gate | up rows in one ffn_up matrix
            return [(f"{p}.ffn_up.weight", "matrix", (H, 2 * c.ffn)), (f"{p}.ffn_down.weight", "matrix", (c.ffn, H))]
        return [(f"{p}.ffn_gate.weight", "matrix", (H, c.ffn)), (f"{p}.ffn_up.weight", "matrix", (H, c.ffn)), (f"{p}.ffn_down.weight", "matrix", (c.ffn, H))]

    post = "post_attention_norm" if (c.arch == "gpt-oss" or c.is_hybrid) else "ffn_norm"
    n_blocks = c.n_layers + (c.nextn_predict_layers if c.is_hybrid else 0)
    for l in range(n_blocks):
        p = f"blk.{l}"
        out.append((f"{p}.attn_norm.weight", "norm", (H,)))
        is_mtp = l >= c.n_layers
        out += attention(p) if (is_mtp or c.layer_is_full_attention(l)) else linear_attention(p)
        out.append((f"{p}.{post}.weight", "norm", (H,)))
        out += ffn(p)
        if is_mtp:
            out += [(f"{p}.nextn.eh_proj.weight", "matrix", (2 * H, H)), (f"{p}.nextn.enorm.weight", "norm", (H,)),
                    (f"{p}.nextn.hnorm.weight", "norm", (H,)), (f"{p}.nextn.shared_head_norm.weight", "norm", (H,))]
    return out


def _gemma4_plan(c: ModelConfig) -> list:
    """Gemma-4 tensors (src/model/gemma4.cpp:160-290): per-layer head geometry, no attn_v on the global layers (V is the raw K
    projection), sandwich norms, a dense GeGLU FFN on every layer and, on MoE checkpoints, a routed path with a fused gate|up bank."""
    H, out = c.hidden, []
    for l in range(c.n_layers):
        p = f"blk.{l}"
        hd, n_kv, _, _ = c.layer_geometry(l)
        out += [(f"{p}.attn_norm.weight", "norm", (H,)), (f"{p}.attn_q.weight", "matrix", (H, c.n_heads * hd)),
                (f"{p}.attn_k.weight", "matrix", (H, n_kv * hd))]
        if c.layer_swa[l]:
            out.append((f"{p}.attn_v.weight", "matrix", (H, n_kv * hd)))
        out += [(f"{p}.attn_output.weight", "matrix", (c.n_heads * hd, H)), (f"{p}.attn_q_norm.weight", "qnorm", (hd,)),
                (f"{p}.attn_k_norm.weight", "norm", (hd,)), (f"{p}.post_attention_norm.weight", "norm", (H,)),
                (f"{p}.ffn_norm.weight", "norm", (H,)), (f"{p}.ffn_gate.weight", "matrix", (H, c.ffn)), (f"{p}.ffn_up.weight", "matrix", (H, c.ffn)),
                (f"{p}.ffn_down.weight", "matrix", (c.ffn, H)), (f"{p}.post_ffw_norm.weight", "norm", (H,)),
                (f"{p}.layer_output_scale.weight", "norm", (1,))]
        if c.is_moe:
            E, F = c.n_experts, c.expert_ffn
            out += [(f"{p}.ffn_gate_inp.weight", "router_sharp", (H, E)), (f"{p}.ffn_gate_inp.scale", "norm", (H,)),
                    (f"{p}.pre_ffw_norm_2.weight", "norm", (H,)), (f"{p}.post_ffw_norm_1.weight", "norm", (H,)),
                    (f"{p}.post_ffw_norm_2.weight", "norm", (H,)), (f"{p}.ffn_gate_up_exps.weight", "expert", (H, 2 * F, E)),
                    (f"{p}.ffn_down_exps.weight", "expert", (F, H, E)), (f"{p}.ffn_down_exps.scale", "norm", (E,))]
    return out


def _matrix_type(name: str, kind: str, K: int, quant: str, n_layers: int) -> int:
    from ..models.sources import _N_LAYERS_HINT, default_policy
    from ..ops.weights import WFormat
    if kind in ("router", "router_sharp"):
        return GGMLType.F32
    _N_LAYERS_HINT["n"] = n_layers
    fmt = default_policy("", quant)(name)
    if fmt == WFormat.EXL3:
        return GGMLType.EXL3 if kind == "matrix" else GGMLType.BF16        # expert stacks stay dense
    t = {WFormat.BF16: GGMLType.BF16, WFormat.Q8: GGMLType.Q8_0, WFormat.Q4K: GGMLType.Q4_K, WFormat.Q6K: GGMLType.Q6_K, WFormat.MXFP4: GGMLType.MXFP4}[fmt]
    if K % block_elems(t):
        t = GGMLType.Q8_0 if K % 32 == 0 else GGMLType.F16
    return t


def _rng(name: str, seed: int) -> np.random.Generator:
    return np.random.default_rng((zlib.crc32(name.encode()) << 16) ^ seed)


def _payload(name: str, kind: str, dims: tuple, ttype: int, seed: int) -> Callable[[], np.ndarray]:
    def make():
        g = _rng(name, seed)
        n = int(np.prod(dims))
        if kind == "norm":
            return (1.0 + 0.05 * g.standard_normal(n)).astype(np.float32)
        if kind == "qnorm":      # Gemma-4 attends with scale 1 on RMS-normalised q and k: a small q gain keeps random-init scores moderate
            return (0.25 + 0.02 * g.standard_normal(n)).astype(np.float32)
        if kind == "ssm_a":
            return (-np.exp(0.5 * g.standard_normal(n))).astype(np.float32)
        if kind == "vector":
            return (0.02 * g.standard_normal(n)).astype(np.float32)
        if kind == "conv":
            return (0.3 * g.standard_normal(n)).astype(np.float32)
        rows = n // dims[0]
        if ttype == GGMLType.F32:
            # Gemma-4 feeds its router rms(x) / sqrt(H): unit-scale weights give logits of order one (decisive routing)
            return ((2.0 if kind == "router_sharp" else 0.02) * g.standard_normal(n)).astype(np.float32)
        step = max(1, (1 << 24) // dims[0])            # quantise in slabs of <= 16 M elements
        out = []
        for r0 in range(0, rows, step):
            x = (0.02 * g.standard_normal((min(step, rows - r0), dims[0]))).astype(np.float32)
            if ttype == GGMLType.F16:
                out.append(x.astype(np.float16).view(np.uint8).reshape(-1))
            elif ttype == GGMLType.BF16:
                out.append((x.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(-1))
            else:
                out.append(quantize(x, ttype))
        return np.concatenate(out)
    return make


def _add_exl3(w, name: str, dims: tuple, quant: str, seed: int) -> int:
    """A random EXL3 layer the way an imported checkpoint stores it: the trellis verbatim as type 37 with dims {16*bits, N/16, K/16} and the
    sign / scale vectors as F16 siblings (src/loaders/hf_import.cpp:553-560).  Any bit stream is a valid trellis."""
    from .exl3 import CODEBOOK_STD
    K, N = dims
    bits = int(quant[5:]) if quant.startswith("exl3-") else 4
    root = name[:-len(".weight")]

    def trellis():
        return _rng(name, seed).integers(0, 256, size=(K // 16) * (N // 16) * 16 * bits * 2, dtype=np.uint8)

    def vec(tag, n, scale):
        def make():
            g = _rng(root + tag, seed)
            return ((g.integers(0, 2, size=n) * 2 - 1) * scale * (1.0 + 0.1 * g.random(n))).astype(np.float16).view(np.uint8).reshape(-1)
        return make

    w.add_tensor(name, (16 * bits, N // 16, K // 16), int(GGMLType.EXL3), trellis)
    w.add_tensor(root + ".suh", (K,), int(GGMLType.F16), vec(".suh", K, 1.0))
    w.add_tensor(root + ".svh", (N,), int(GGMLType.F16), vec(".svh", N, 0.02 / CODEBOOK_STD))
    return 3


def write_synthetic_gguf(cfg: ModelConfig, path: str, quant: str = "q8_0", seed: int = 0, tokenizer: bool = True,
                         extra_kv: Iterable = ()) -> dict:
    """Writes the checkpoint; returns {"tensors": n, "bytes": payload bytes}."""
    w = GGUFWriter()
    kv = config_to_kv(cfg)
    if tokenizer:
        kv.update(synthetic_tokenizer_kv(cfg))
    else:
        kv[f"{cfg.arch}.vocab_size"] = cfg.vocab
    kv["general.file_type"] = {"q8_0": 7, "q4_k_m": 15, "mxfp4": 38, "bf16": 32}.get(quant, 0)
    kv["general.quantization_version"] = 2
    for k, v in extra_kv:
        kv[k] = v
    for k, v in kv.items():
        w.add_kv(k, v)
    n = 0
    for name, kind, dims in tensor_plan(cfg):
        t = _matrix_type(name, kind, dims[0], quant, cfg.n_layers) if kind in ("matrix", "expert", "router", "router_sharp") else GGMLType.F32
        if t == GGMLType.EXL3:
            if dims[0] % 128 or dims[1] % 128:
                t = GGMLType.BF16          # the 128-point rotations need multiples of 128 on both sides
            else:
                n += _add_exl3(w, name, dims, quant, seed)
                continue
        w.add_tensor(name, dims, int(t), _payload(name, kind, dims, int(t), seed))
        n += 1
    w.write(path)
    import os
    return {"tensors": n, "bytes": os.path.getsize(path)}


def assistant_tensor_plan(a) -> list:
    """Tensors of a ``gemma4-assistant`` head file (src/model/gemma4_assistant.cpp:75-150); ``a`` is an
    ``models.gemma4_assistant.AssistantConfig``."""
    H, BB = a.hidden, a.backbone
    out = [("token_embd.weight", "matrix", (H, a.vocab)), ("output_norm.weight", "norm", (H,)),
           ("nextn.pre_projection.weight", "matrix", (2 * BB, H)), ("nextn.post_projection.weight", "matrix", (H, BB))]
    for l in range(a.n_layers):
        p, hd = f"blk.{l}", a.head_dim[l]
        out += [(f"{p}.attn_norm.weight", "norm", (H,)), (f"{p}.attn_q_norm.weight", "qnorm", (hd,)),
                (f"{p}.post_attention_norm.weight", "norm", (H,)), (f"{p}.ffn_norm.weight", "norm", (H,)),
                (f"{p}.post_ffw_norm.weight", "norm", (H,)), (f"{p}.layer_output_scale.weight", "norm", (1,)),
                (f"{p}.attn_q.weight", "matrix", (H, a.n_q_heads * hd)), (f"{p}.attn_output.weight", "matrix", (a.n_q_heads * hd, H)),
                (f"{p}.ffn_gate.weight", "matrix", (H, a.ffn)), (f"{p}.ffn_up.weight", "matrix", (H, a.ffn)), (f"{p}.ffn_down.weight", "matrix", (a.ffn, H))]
    return out


def write_synthetic_assistant_gguf(a, path: str, quant: str = "q8_0", seed: int = 0) -> dict:
    """Random-init ``gemma4-assistant`` head for a Gemma-4 target (``a``: AssistantConfig), with the metadata keys its loader reads."""
    w = GGUFWriter()
    k = lambda s: f"gemma4-assistant.{s}"
    swa = [i for i, s in enumerate(a.is_swa) if s]
    glb = [i for i, s in enumerate(a.is_swa) if not s]
    kv = {"general.architecture": "gemma4-assistant", "general.name": "synthetic gemma4 assistant head", k("block_count"): a.n_layers,
          k("embedding_length"): a.hidden, k("feed_forward_length"): a.ffn, k("attention.head_count"): a.n_q_heads,
          k("attention.head_count_kv"): [int(v) for v in a.n_kv_heads], k("attention.layer_norm_rms_epsilon"): float(a.rms_eps),
          k("attention.sliding_window"): a.sliding_window, k("attention.sliding_window_pattern"): [bool(s) for s in a.is_swa]}
    if glb:
        kv.update({k("attention.key_length"): a.head_dim[glb[0]], k("rope.dimension_count"): a.n_rot[glb[0]], k("rope.freq_base"): float(a.rope_theta[glb[0]])})
    if swa:
        kv.update({k("attention.key_length_swa"): a.head_dim[swa[0]], k("rope.dimension_count_swa"): a.n_rot[swa[0]],
                   k("rope.freq_base_swa"): float(a.rope_theta[swa[0]])})
    for key, v in kv.items():
        w.add_kv(key, v)
    n = 0
    for name, kind, dims in assistant_tensor_plan(a):
        t = _matrix_type(name, kind, dims[0], quant, a.n_layers) if kind == "matrix" else GGMLType.F32
        w.add_tensor(name, dims, int(t), _payload("assistant." + name, kind, dims, int(t), seed))
        n += 1
    w.write(path)
    import os
    return {"tensors": n, "bytes": os.path.getsize(path)}
