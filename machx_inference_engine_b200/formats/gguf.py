"""GGUF v3 files: zero-copy reader (split shards merged) and streaming writer.

Thin Python faces over the C++ container code in ``csrc/host/gguf.cpp``.
Reference parity: include/ie/gguf.hpp:49-132 (reader API), include/ie/gguf_writer.hpp:21-74.
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass
from enum import IntEnum
from typing import Any, Iterable

import numpy as np

from .. import _lib


class GGMLType(IntEnum):
    """Tensor type ids; equal to ggml's (reference: include/ie/dtype.hpp:15-57)."""
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q8_0 = 8
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    I8 = 24
    I16 = 25
    I32 = 26
    I64 = 27
    F64 = 28
    BF16 = 30
    EXL3 = 37        # this engine family's id for a verbatim EXL3 trellis (int16 words; dims {16*bits, N/16, K/16})
    MXFP4 = 39


def block_elems(t: int) -> int:
    return _lib.host().mx_type_block_elems(int(t))


def block_bytes(t: int) -> int:
    return _lib.host().mx_type_block_bytes(int(t))


def bytes_for(t: int, n: int) -> int:
    return _lib.host().mx_bytes_for(int(t), int(n))


def type_name(t: int) -> str:
    return _lib.host().mx_type_name(int(t)).decode() or f"type{int(t)}"


@dataclass
class GGUFTensor:
    name: str
    dims: tuple[int, ...]      # ggml order: dims[0] is the contiguous (input) dimension
    type: int
    nbytes: int
    shard: int
    index: int
    _reader: "GGUFReader"

    @property
    def shape(self) -> tuple[int, ...]:
        """Row-major (torch/numpy) shape: ggml dims reversed."""
        return tuple(reversed(self.dims))

    @property
    def n_elements(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    def raw(self) -> np.ndarray:
        """uint8 view of the payload inside the mapping (no copy; valid while the reader is open)."""
        ptr = _lib.host().mx_gguf_tensor_ptr(self._reader._h, self.index)
        if not ptr:
            raise KeyError(self.name)
        buf = (C.c_uint8 * self.nbytes).from_address(ptr)
        arr = np.frombuffer(buf, dtype=np.uint8)
        arr.flags.writeable = False
        return arr

    def to_float32(self) -> np.ndarray:
        """Dequantised copy with the row-major shape."""
        from . import quant
        return quant.dequantize(self.raw(), self.type, self.n_elements).reshape(self.shape)


class GGUFReader:
    def __init__(self, path: str):
        lib = _lib.host()
        self._h = lib.mx_gguf_open(str(path).encode())
        if not self._h:
            raise ValueError(_lib.host_error())
        n = lib.mx_gguf_meta_json_len(self._h)
        doc = json.loads(C.string_at(lib.mx_gguf_meta_json(self._h), n).decode("utf-8", "replace"))
        self.version: int = doc["version"]
        self.kv: dict[str, Any] = doc["kv"]
        self.shards: list[str] = doc["shards"]
        self.tensors: dict[str, GGUFTensor] = {}
        for i, t in enumerate(doc["tensors"]):
            self.tensors[t["name"]] = GGUFTensor(t["name"], tuple(t["dims"]), t["type"], t["nbytes"], t["shard"], i, self)

    def close(self) -> None:
        if self._h:
            _lib.host().mx_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def get(self, key: str, default: Any = None) -> Any:
        return self.kv.get(key, default)

    def has_tensor(self, name: str) -> bool:
        return name in self.tensors

    def tensor(self, name: str) -> GGUFTensor:
        return self.tensors[name]

    @property
    def total_tensor_bytes(self) -> int:
        return sum(t.nbytes for t in self.tensors.values())


class GGUFWriter:
    """Declare metadata and tensors, then stream payloads in declaration order.

    Only one tensor payload needs to be resident at a time (the streaming mode of the
    reference's writer); ``add_tensor`` takes either bytes-like data or a zero-argument
    callable that produces it when its turn comes.
    """

    def __init__(self) -> None:
        self._lib = _lib.host()
        self._w = self._lib.mx_ggufw_new()
        self._payloads: list[Any] = []
        self._sizes: list[int] = []

    def add_kv(self, key: str, value: Any) -> None:
        k = key.encode()
        L = self._lib
        if isinstance(value, bool):
            L.mx_ggufw_kv_bool(self._w, k, int(value))
        elif isinstance(value, int):
            if value < 0:
                L.mx_ggufw_kv_i32(self._w, k, value)
            elif value >= 2**32:
                L.mx_ggufw_kv_u64(self._w, k, value)
            else:
                L.mx_ggufw_kv_u32(self._w, k, value)
        elif isinstance(value, float):
            L.mx_ggufw_kv_f32(self._w, k, value)
        elif isinstance(value, (str, bytes)):
            b = value.encode() if isinstance(value, str) else value
            L.mx_ggufw_kv_str(self._w, k, b, len(b))
        elif isinstance(value, (list, tuple, np.ndarray)):
            self._add_array(k, value)
        else:
            raise TypeError(f"unsupported GGUF metadata value for {key}: {type(value)}")

    def _add_array(self, k: bytes, value: Iterable) -> None:
        L = self._lib
        vals = list(value)
        if vals and isinstance(vals[0], (str, bytes)):
            bs = [v.encode() if isinstance(v, str) else v for v in vals]
            blob = b"".join(bs)
            lens = np.array([len(b) for b in bs], dtype=np.uint64)
            L.mx_ggufw_kv_arr_str(self._w, k, blob, lens.ctypes.data, len(bs))
        elif vals and isinstance(vals[0], (float, np.floating)):
            a = np.asarray(vals, dtype=np.float32)
            L.mx_ggufw_kv_arr_f32(self._w, k, a.ctypes.data, a.size)
        else:
            a = np.asarray(vals, dtype=np.int32)
            L.mx_ggufw_kv_arr_i32(self._w, k, a.ctypes.data, a.size)

    def add_tensor(self, name: str, dims: Iterable[int], ttype: int, data: Any) -> None:
        """``dims`` in ggml order (contiguous dimension first)."""
        d = np.asarray(list(dims), dtype=np.uint64)
        nb = self._lib.mx_ggufw_add_tensor(self._w, name.encode(), len(d), d.ctypes.data, int(ttype))
        if nb == 0 and int(np.prod(d)) != 0:
            raise ValueError(_lib.host_error())
        self._payloads.append(data)
        self._sizes.append(nb)

    def write(self, path: str) -> None:
        L = self._lib
        try:
            if L.mx_ggufw_begin(self._w, str(path).encode()) != 0:
                raise IOError(_lib.host_error())
            for data, nb in zip(self._payloads, self._sizes):
                if callable(data):
                    data = data()
                arr = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data)
                arr = arr.view(np.uint8).reshape(-1)
                if arr.size != nb:
                    raise ValueError(f"tensor payload is {arr.size} bytes, expected {nb}")
                if L.mx_ggufw_write(self._w, arr.ctypes.data, nb) != 0:
                    raise IOError(_lib.host_error())
            if L.mx_ggufw_end(self._w) != 0:
                raise IOError(_lib.host_error())
        finally:
            L.mx_ggufw_free(self._w)
            self._w = None
            self._payloads = []
