"""Tokenizer front end over the C++ implementation (``csrc/host/tokenizer.cpp``).

Reference parity: ``Tokenizer::{load_from_gguf, encode, decode}`` (include/ie/tokenizer.hpp,
src/tokenizer/tokenizer.cpp:80-196,579-726): vocabulary, merges, token types and scores come from
the GGUF ``tokenizer.ggml.*`` keys; ``tokenizer.ggml.pre`` picks the pre-tokenizer; llama-bpe / tekken
files default ``add_bos_token`` to true.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, Mapping, Optional, Sequence

import numpy as np

from .. import _lib

_PRE = {"qwen2": 0, "default": 0, "llama-bpe": 1, "llama3": 1, "dbrx": 1, "tekken": 2, "gpt-4o": 2, "o200k": 2, "gpt-2": 3, "gpt2": 3}


def _declare(lib):
    if getattr(lib, "_tok_declared", False):
        return
    vp, cp, u64, i32, i64 = C.c_void_p, C.c_char_p, C.c_uint64, C.c_int32, C.c_int64
    lib.mx_tok_create.restype = vp
    lib.mx_tok_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, cp, vp, u64, vp, vp, cp, vp, u64]
    lib.mx_tok_free.argtypes = [vp]
    lib.mx_tok_find.restype = i32
    lib.mx_tok_find.argtypes = [vp, cp, u64]
    lib.mx_tok_is_special.argtypes = [vp, i32]
    lib.mx_tok_encode.restype = i64
    lib.mx_tok_encode.argtypes = [vp, cp, u64, C.c_int, vp, u64]
    lib.mx_tok_decode.restype = i64
    lib.mx_tok_decode.argtypes = [vp, vp, u64, C.c_int, vp, u64, vp, u64]
    lib._tok_declared = True


class Tokenizer:
    def __init__(self, tokens: Sequence, merges: Sequence = (), token_types: Optional[Sequence[int]] = None,
                 scores: Optional[Sequence[float]] = None, model: str = "gpt2", pre: str = "qwen2", bos_id: int = -1, eos_id: int = -1,
                 pad_id: int = -1, add_bos: Optional[bool] = None, add_space_prefix: bool = True, chat_template: str = ""):
        self._lib = _lib.host()
        _declare(self._lib)
        toks = [t.encode("utf-8", "surrogateescape") if isinstance(t, str) else bytes(t) for t in tokens]
        mer = [m.encode("utf-8", "surrogateescape") if isinstance(m, str) else bytes(m) for m in merges]
        tl = np.array([len(t) for t in toks], dtype=np.uint64)
        ml = np.array([len(m) for m in mer], dtype=np.uint64)
        ty = np.asarray(token_types, dtype=np.int32) if token_types is not None and len(token_types) == len(toks) else None
        sc = np.asarray(scores, dtype=np.float32) if scores is not None and len(scores) == len(toks) else None
        self.model = model
        kind = {"gpt2": 0, "llama": 1, "gemma": 2}.get(model, 0)
        self.pre = pre
        ignore_merges = pre in ("llama-bpe", "llama3", "dbrx", "tekken")
        self._h = self._lib.mx_tok_create(kind, _PRE.get(pre, 0), int(ignore_merges), int(add_space_prefix), b"".join(toks), tl.ctypes.data, len(toks),
                                          ty.ctypes.data if ty is not None else None, sc.ctypes.data if sc is not None else None,
                                          b"".join(mer), ml.ctypes.data if len(mer) else None, len(mer))
        self.vocab_size = len(toks)
        self._tokens = toks
        self.bos_id, self.eos_id, self.pad_id = bos_id, eos_id, pad_id
        if add_bos is None:
            add_bos = pre in ("llama-bpe", "llama3", "tekken") or model == "llama"
        self.add_bos = bool(add_bos) and bos_id >= 0
        self.chat_template = chat_template

    @classmethod
    def from_gguf_kv(cls, kv: Mapping) -> "Tokenizer":
        toks = kv.get("tokenizer.ggml.tokens")
        if toks is None:
            raise ValueError("GGUF has no tokenizer.ggml.tokens")
        model = str(kv.get("tokenizer.ggml.model", "gpt2"))
        arch = str(kv.get("general.architecture", ""))
        if arch.startswith("gemma") and model != "gpt2":
            model = "gemma"
        add_bos = kv.get("tokenizer.ggml.add_bos_token")
        return cls(toks, kv.get("tokenizer.ggml.merges") or (), kv.get("tokenizer.ggml.token_type"), kv.get("tokenizer.ggml.scores"), model=model,
                   pre=str(kv.get("tokenizer.ggml.pre", "qwen2")), bos_id=int(kv.get("tokenizer.ggml.bos_token_id", -1)),
                   eos_id=int(kv.get("tokenizer.ggml.eos_token_id", -1)), pad_id=int(kv.get("tokenizer.ggml.padding_token_id", -1)),
                   add_bos=None if add_bos is None else bool(add_bos), add_space_prefix=bool(kv.get("tokenizer.ggml.add_space_prefix", True)),
                   chat_template=str(kv.get("tokenizer.chat_template", "")))

    def __del__(self):  # pragma: no cover
        try:
            if self._h:
                self._lib.mx_tok_free(self._h)
        except Exception:
            pass

    def find_token(self, s: str) -> int:
        b = s.encode()
        return self._lib.mx_tok_find(self._h, b, len(b))

    def is_special(self, tid: int) -> bool:
        return bool(self._lib.mx_tok_is_special(self._h, int(tid)))

    def token_bytes(self, tid: int) -> bytes:
        return self._tokens[tid]

    def encode(self, text: str, allow_special: bool = True, add_bos: Optional[bool] = None) -> list:
        b = text.encode("utf-8", "surrogateescape")
        cap = max(16, len(b) + 8)
        buf = np.empty(cap, dtype=np.int32)
        n = self._lib.mx_tok_encode(self._h, b, len(b), int(allow_special), buf.ctypes.data, cap)
        if n > cap:
            buf = np.empty(n, dtype=np.int32)
            n = self._lib.mx_tok_encode(self._h, b, len(b), int(allow_special), buf.ctypes.data, n)
        ids = buf[:n].tolist()
        if (self.add_bos if add_bos is None else add_bos) and self.bos_id >= 0 and (not ids or ids[0] != self.bos_id):
            ids.insert(0, self.bos_id)
        return ids

    def decode_bytes(self, ids: Iterable[int], skip_special: bool = False, keep_special: Iterable[int] = ()) -> bytes:
        a = np.asarray(list(ids), dtype=np.int32)
        k = np.asarray(list(keep_special), dtype=np.int32)
        cap = max(64, 16 * len(a) + 64)
        buf = C.create_string_buffer(cap)
        n = self._lib.mx_tok_decode(self._h, a.ctypes.data, len(a), int(skip_special), k.ctypes.data if len(k) else None, len(k), buf, cap)
        if n > cap:
            buf = C.create_string_buffer(n)
            n = self._lib.mx_tok_decode(self._h, a.ctypes.data, len(a), int(skip_special), k.ctypes.data if len(k) else None, len(k), buf, n)
        return buf.raw[:n]

    def decode(self, ids: Iterable[int], skip_special: bool = False, keep_special: Iterable[int] = ()) -> str:
        return self.decode_bytes(ids, skip_special, keep_special).decode("utf-8", "replace")


class IncrementalDetokenizer:
    """Streams text for a growing id list without ever splitting a UTF-8 sequence
    (the reference's incremental, UTF-8-boundary-safe detokenise step: src/engine/engine.cpp:804-869)."""

    def __init__(self, tok: Tokenizer, skip_special: bool = True, keep_special: Iterable[int] = ()):
        self.tok, self.skip, self.keep = tok, skip_special, tuple(keep_special)
        self.pending = b""

    def push(self, tid: int) -> str:
        self.pending += self.tok.decode_bytes([tid], self.skip, self.keep)
        cut = utf8_safe_prefix(self.pending)
        out, self.pending = self.pending[:cut], self.pending[cut:]
        return out.decode("utf-8", "replace")

    def flush(self) -> str:
        out, self.pending = self.pending, b""
        return out.decode("utf-8", "replace")


def utf8_safe_prefix(b: bytes) -> int:
    """Length of the longest prefix of ``b`` that does not end inside a multi-byte UTF-8 sequence."""
    n = len(b)
    i = n - 1
    back = 0
    while i >= 0 and back < 4 and (b[i] & 0xC0) == 0x80:
        i -= 1
        back += 1
    if i < 0:
        return n if back == 0 else 0
    lead = b[i]
    need = 1 if lead < 0x80 else 2 if (lead >> 5) == 6 else 3 if (lead >> 4) == 14 else 4 if (lead >> 3) == 30 else 1
    return n if back + 1 >= need else i
