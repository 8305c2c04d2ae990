"""``ie import``: Hugging Face checkpoint directory (safetensors; plain fp16/bf16, AWQ or GPTQ 4-bit) -> GGUF.

Reference parity: src/loaders/hf_import.cpp:25-438 (``parse_hf_config``, ``hf_to_gguf_tensor_name``, ``import_awq_to_gguf``:
projections -> Q4_K, embeddings and other 2-D tensors -> Q6_K, 1-D tensors and biases -> F32, tokenizer metadata copied from
a reference GGUF and padded to the embedding rows, streaming output).  Extensions: the tokenizer can also be taken from the
checkpoint's own ``tokenizer.json``; un-quantised checkpoints import through the same recipe; llama-architecture Q/K rows
are written in the interleaved order GGUF files of that family use.  Dense llama / qwen2 / qwen3 / mistral checkpoints.
"""
from __future__ import annotations

import json
import os
import sys
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

from .gguf import GGMLType, GGUFReader, GGUFWriter
from .quant import quantize
from .safetensors import SafetensorsModel, awq_dequant, gptq_dequant


class ImportError_(ValueError):
    pass


@dataclass
class HFMeta:
    arch: str = "llama"
    n_layers: int = 0
    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    ffn: int = 0
    vocab: int = 0
    head_dim: int = 0
    rope_dim: int = 0
    ctx_train: int = 4096
    rope_theta: float = 10000.0
    rms_eps: float = 1e-6
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    quant_method: str = ""           # "" | awq | gptq | exl3
    bits: int = 4
    group_size: int = 128
    version: str = "gemm"
    desc_act: bool = False
    extra: dict = field(default_factory=dict)


def parse_hf_config(text: str) -> HFMeta:
    try:
        c = json.loads(text)
    except Exception as e:
        raise ImportError_(f"config.json parse error: {e}")
    m = HFMeta()
    m.arch = {"mistral": "llama"}.get(c.get("model_type", "llama"), c.get("model_type", "llama"))
    for key, attr in (("num_hidden_layers", "n_layers"), ("hidden_size", "hidden"), ("num_attention_heads", "n_heads"),
                      ("num_key_value_heads", "n_kv_heads"), ("intermediate_size", "ffn"), ("vocab_size", "vocab")):
        if not isinstance(c.get(key), int):
            raise ImportError_(f"config: missing {key}")
        setattr(m, attr, c[key])
    m.head_dim = int(c.get("head_dim") or (m.hidden // m.n_heads))
    m.rope_dim = int(m.head_dim * float(c.get("partial_rotary_factor", 1.0)))
    m.ctx_train = int(c.get("max_position_embeddings", 4096))
    m.rope_theta = float(c.get("rope_theta", 10000.0))
    m.rms_eps = float(c.get("rms_norm_eps", 1e-6))
    m.tie_word_embeddings = bool(c.get("tie_word_embeddings", False))
    m.attention_bias = bool(c.get("attention_bias", False))
    q = c.get("quantization_config")
    if q:
        m.quant_method = str(q.get("quant_method", "")).lower()
        m.bits = int(q.get("bits", q.get("w_bit", 4)))
        m.group_size = int(q.get("group_size", q.get("q_group_size", 128)))
        m.version = str(q.get("version", "gemm")).lower()
        m.desc_act = bool(q.get("desc_act", False))
        if m.quant_method == "exl3":
            # trellis layers carry their own width (bits = trellis.shape[-1] / 16, it may differ per layer); nothing else to parse
            if m.arch not in ("llama",):
                raise ImportError_(f"EXL3 import takes dense llama checkpoints, not '{m.arch}'")
            return m
        if m.quant_method not in ("awq", "gptq"):
            raise ImportError_(f"unsupported quant_method '{m.quant_method}' (awq | gptq | exl3)")
        if m.bits != 4:
            raise ImportError_(f"4-bit only (got {m.bits})")
        if m.quant_method == "awq" and m.version != "gemm":
            raise ImportError_(f"AWQ pack order '{m.version}' is not supported (only 'gemm')")
    if m.arch not in ("llama", "qwen2", "qwen3"):
        raise ImportError_(f"import supports dense llama / mistral / qwen2 / qwen3 checkpoints, not '{m.arch}'")
    return m


_ROLES = {
    "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output",
    "self_attn.q_norm": "attn_q_norm", "self_attn.k_norm": "attn_k_norm", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
    "mlp.down_proj": "ffn_down", "input_layernorm": "attn_norm", "post_attention_layernorm": "ffn_norm",
}
_SUFFIXES = (".weight", ".bias", ".qweight", ".qzeros", ".scales", ".g_idx")


def hf_to_gguf_name(name: str) -> str:
    """'' for tensors that have no GGUF counterpart (rotary caches and the like)."""
    top = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight", "lm_head.weight": "output.weight"}
    if name in top:
        return top[name]
    if not name.startswith("model.layers."):
        return ""
    rest = name[len("model.layers."):]
    layer, _, rest = rest.partition(".")
    if not layer.isdigit():
        return ""
    for s in _SUFFIXES:
        if rest.endswith(s):
            role = _ROLES.get(rest[:-len(s)])
            return f"blk.{layer}.{role}{s}" if role else ""
    return ""


def _llama_permute(w: np.ndarray, n_head: int) -> np.ndarray:
    rows, k = w.shape
    hd = rows // n_head
    return w.reshape(n_head, 2, hd // 2, k).swapaxes(1, 2).reshape(rows, k)


def _tokenizer_kv_from_json(path: str, vocab_rows: int) -> dict:
    """Byte-level BPE ``tokenizer.json`` (Hugging Face tokenizers format) -> tokenizer.ggml.* metadata."""
    tj = json.load(open(path, encoding="utf-8"))
    model = tj.get("model", {})
    if model.get("type") != "BPE":
        raise ImportError_("tokenizer.json: only BPE tokenizers are supported")
    vocab = model["vocab"]
    n = max(max(vocab.values()) + 1, vocab_rows)
    for t in tj.get("added_tokens", []):
        n = max(n, t["id"] + 1)
    tokens = [f"[PAD{i}]" for i in range(n)]
    types = [5] * n                                              # unused until named
    for s, i in vocab.items():
        tokens[i], types[i] = s, 1
    for t in tj.get("added_tokens", []):
        tokens[t["id"]] = t["content"]
        types[t["id"]] = 3 if t.get("special", True) else 4
    merges = [m if isinstance(m, str) else " ".join(m) for m in model.get("merges", [])]
    kv = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.token_type": types, "tokenizer.ggml.merges": merges}
    cfgp = os.path.join(os.path.dirname(path), "tokenizer_config.json")
    pre = "qwen2"
    if os.path.exists(cfgp):
        tc = json.load(open(cfgp, encoding="utf-8"))
        ids = {s: i for i, s in enumerate(tokens)}

        def tok_id(v):
            v = v.get("content") if isinstance(v, dict) else v
            return ids.get(v, -1) if isinstance(v, str) else -1
        for key, name in (("bos_token", "bos_token_id"), ("eos_token", "eos_token_id"), ("pad_token", "padding_token_id")):
            i = tok_id(tc.get(key))
            if i >= 0:
                kv[f"tokenizer.ggml.{name}"] = i
        if isinstance(tc.get("chat_template"), str):
            kv["tokenizer.chat_template"] = tc["chat_template"]
        if "<|begin_of_text|>" in ids:
            pre = "llama-bpe"
    kv["tokenizer.ggml.pre"] = pre
    return kv


def _tokenizer_kv_from_gguf(path: str, vocab_rows: int) -> dict:
    r = GGUFReader(path)
    kv = {k: v for k, v in r.kv.items() if k.startswith("tokenizer.")}
    toks = list(kv.get("tokenizer.ggml.tokens", []))
    if not toks:
        raise ImportError_(f"{path} holds no tokenizer metadata")
    if len(toks) < vocab_rows:          # embedding tables are often padded past the tokenizer's vocabulary
        pad = vocab_rows - len(toks)
        kv["tokenizer.ggml.tokens"] = toks + [f"[PAD{len(toks) + i}]" for i in range(pad)]
        if "tokenizer.ggml.token_type" in kv:
            kv["tokenizer.ggml.token_type"] = list(kv["tokenizer.ggml.token_type"]) + [5] * pad
        if "tokenizer.ggml.scores" in kv:
            kv["tokenizer.ggml.scores"] = list(kv["tokenizer.ggml.scores"]) + [0.0] * pad
    return kv


def _pick_type(name: str, k: int) -> int:
    proj = any(s in name for s in ("attn_q.", "attn_k.", "attn_v.", "attn_output.", "ffn_gate.", "ffn_up.", "ffn_down."))
    want = GGMLType.Q4_K if proj else GGMLType.Q6_K
    if k % 256:
        want = GGMLType.Q8_0 if k % 32 == 0 else GGMLType.F16
    return int(want)


def _add_exl3_tensors(w: GGUFWriter, st: SafetensorsModel, names: list, m: HFMeta) -> int:
    """An EXL3 (exllamav3) checkpoint: every quantised linear is ``<module>.trellis`` int16 [K/16, N/16, 16*bits] with ``.suh`` [K] and
    ``.svh`` [N]; they go into the GGUF unchanged (type 37, dims {16*bits, N/16, K/16}, and F16 siblings ``<name>.suh`` / ``.svh``), the
    embedding stays F16, vectors become F32.  Q / K rows keep the Hugging Face order (the graph skips its llama re-ordering for these
    layers).  Only the default codebook is handled: a layer with ``mcg`` / ``mul1`` tensors, or with the legacy packed ``su`` / ``sv``
    sign fields, is refused.  Reference parity: src/loaders/hf_import.cpp:440-592."""
    n_t = 0
    for n in sorted(names, key=lambda s: (hf_to_gguf_name(s.replace(".trellis", ".weight")) or "~" + s)):
        if n.endswith((".suh", ".svh")):
            continue
        if n.endswith((".mcg", ".mul1", ".su", ".sv")):
            raise ImportError_(f"{n}: only EXL3 layers with the default codebook and fp16 suh / svh vectors are supported")
        if n.endswith(".trellis"):
            base = n[:-len(".trellis")]
            g = hf_to_gguf_name(base + ".weight")
            if not g:
                continue
            shp = st.shape(n)
            if len(shp) != 3 or shp[2] % 16 or not 1 <= shp[2] // 16 <= 8:
                raise ImportError_(f"{n}: trellis shape {tuple(shp)} is not [K/16, N/16, 16*bits]")
            if not (st.has(base + ".suh") and st.has(base + ".svh")):
                raise ImportError_(f"{base}: EXL3 layer is missing suh / svh")
            tk, tn, wb = (int(v) for v in shp)
            if (tk * 16) % 128 or (tn * 16) % 128 or st.shape(base + ".suh")[0] != tk * 16 or st.shape(base + ".svh")[0] != tn * 16:
                raise ImportError_(f"{base}: EXL3 layer shapes do not fit ({tk * 16} x {tn * 16})")
            root = g[:-len(".weight")]
            w.add_tensor(g, [wb, tn, tk], int(GGMLType.EXL3), (lambda nn=n: np.ascontiguousarray(st.numpy(nn)).view(np.uint8).reshape(-1)))
            for tag in (".suh", ".svh"):
                w.add_tensor(root + tag, [int(st.shape(base + tag)[0])], int(GGMLType.F16),
                             (lambda nn=base + tag: st.float32(nn).astype(np.float16).view(np.uint8).reshape(-1)))
            n_t += 3
            continue
        g = hf_to_gguf_name(n)
        if not g or (m.tie_word_embeddings and g == "output.weight"):
            continue
        shp = st.shape(n)
        if len(shp) == 2:
            w.add_tensor(g, [int(shp[1]), int(shp[0])], int(GGMLType.F16), (lambda nn=n: st.float32(nn).astype(np.float16).view(np.uint8).reshape(-1)))
        else:
            w.add_tensor(g, [int(np.prod(shp))], int(GGMLType.F32), (lambda nn=n: st.float32(nn).astype(np.float32).reshape(-1)))
        n_t += 1
    return n_t


def import_to_gguf(hf_dir: str, out_path: str, tokenizer_gguf: Optional[str] = None, stream: bool = True, log=None) -> dict:
    log = log or (lambda s: print(s, file=sys.stderr))
    cfg_path = os.path.join(hf_dir, "config.json")
    if not os.path.exists(cfg_path):
        raise ImportError_(f"{hf_dir} has no config.json")
    m = parse_hf_config(open(cfg_path).read())
    st = SafetensorsModel(hf_dir)
    names = list(st.names())
    arch = m.arch
    w = GGUFWriter()
    kv = {
        "general.architecture": arch, "general.name": os.path.basename(os.path.normpath(hf_dir)), f"{arch}.block_count": m.n_layers,
        f"{arch}.embedding_length": m.hidden, f"{arch}.attention.head_count": m.n_heads, f"{arch}.attention.head_count_kv": m.n_kv_heads,
        f"{arch}.feed_forward_length": m.ffn, f"{arch}.attention.key_length": m.head_dim, f"{arch}.attention.value_length": m.head_dim,
        f"{arch}.rope.dimension_count": m.rope_dim, f"{arch}.context_length": m.ctx_train, f"{arch}.rope.freq_base": float(m.rope_theta),
        f"{arch}.attention.layer_norm_rms_epsilon": float(m.rms_eps), "general.file_type": 15, "general.quantization_version": 2,
    }
    emb_rows = st.shape("model.embed_tokens.weight")[0]
    tj = os.path.join(hf_dir, "tokenizer.json")
    if tokenizer_gguf:
        kv.update(_tokenizer_kv_from_gguf(tokenizer_gguf, emb_rows))
    elif os.path.exists(tj):
        kv.update(_tokenizer_kv_from_json(tj, emb_rows))
    else:
        raise ImportError_("no tokenizer: pass --tokenizer-gguf <file.gguf> or put tokenizer.json next to the weights")
    for k, v in kv.items():
        w.add_kv(k, v)

    if m.quant_method == "exl3":
        n_t = _add_exl3_tensors(w, st, names, m)
        w.write(out_path)
        log(f"[import] {n_t} tensors -> {out_path} ({os.path.getsize(out_path) / 1e6:.1f} MB), quant source: exl3 (trellis layers kept verbatim)")
        return {"tensors": n_t, "arch": arch, "bytes": os.path.getsize(out_path)}

    # group the quantised triplets by module
    plan, done = [], set()
    for n in sorted(names, key=lambda s: (hf_to_gguf_name(s) or "~" + s)):
        g = hf_to_gguf_name(n)
        if not g or n in done:
            continue
        if n.endswith((".qzeros", ".scales", ".g_idx")):
            continue
        if n.endswith(".qweight"):
            base = n[:-len(".qweight")]
            for part in (".qzeros", ".scales"):
                if not st.has(base + part):
                    raise ImportError_(f"{base}: quantised module is missing {part}")
            in_f, out_f = (st.shape(n)[0], st.shape(n)[1] * 8) if m.quant_method == "awq" else (st.shape(n)[0] * 8, st.shape(n)[1])
            plan.append((g[:-len(".qweight")] + ".weight", "q", base, (in_f, out_f)))
        elif len(st.shape(n)) == 2:
            plan.append((g, "dense", n, (st.shape(n)[1], st.shape(n)[0])))
        else:
            plan.append((g, "vec", n, st.shape(n)))
    if m.tie_word_embeddings:
        plan = [p for p in plan if p[0] != "output.weight"]

    def make(gname, kind, src, dims):
        def f():
            if kind == "vec":
                return st.float32(src).astype(np.float32).reshape(-1)
            if kind == "q":
                if m.quant_method == "awq":
                    dense = awq_dequant(st.numpy(src + ".qweight"), st.numpy(src + ".qzeros"), st.numpy(src + ".scales"), m.group_size)
                else:
                    gi = st.numpy(src + ".g_idx") if (m.desc_act and st.has(src + ".g_idx")) else None
                    dense = gptq_dequant(st.numpy(src + ".qweight"), st.numpy(src + ".qzeros"), st.numpy(src + ".scales"), m.group_size, gi)
            else:
                dense = st.float32(src)
            if arch == "llama" and (".attn_q." in gname or ".attn_k." in gname):
                dense = _llama_permute(dense, m.n_heads if ".attn_q." in gname else m.n_kv_heads)
            t = _pick_type(gname, dense.shape[1])
            if t == GGMLType.F16:
                return dense.astype(np.float16).view(np.uint8).reshape(-1)
            return quantize(np.ascontiguousarray(dense), t)
        return f

    n_t = 0
    for gname, kind, src, dims in plan:
        if kind == "vec":
            w.add_tensor(gname, [int(np.prod(dims))], int(GGMLType.F32), make(gname, kind, src, dims))
        else:
            k, n_out = dims
            f = make(gname, kind, src, dims)
            w.add_tensor(gname, [k, n_out], _pick_type(gname, k), f if stream else f())
        n_t += 1
    w.write(out_path)
    log(f"[import] {n_t} tensors -> {out_path} ({os.path.getsize(out_path) / 1e6:.1f} MB), quant source: {m.quant_method or 'none'}")
    return {"tensors": n_t, "arch": arch, "bytes": os.path.getsize(out_path)}
