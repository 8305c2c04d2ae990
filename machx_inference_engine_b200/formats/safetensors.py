"""safetensors files: memory-mapped reader (single file or a sharded directory with ``model.safetensors.index.json``)
and a small writer used by the import tests.  The container code (mmap, header bounds checks) is C++
(``csrc/host/hfimport.cpp``); reference parity: include/ie/safetensors.hpp:30-92."""
from __future__ import annotations

import ctypes as C
import glob
import json
import os
import struct
from typing import Iterable

import numpy as np

from .. import _lib

_DT = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64, "I32": np.int32, "I16": np.int16,
       "I8": np.int8, "U8": np.uint8, "BOOL": np.uint8, "U16": np.uint16, "U32": np.uint32}


def _lib_st():
    lib = _lib.host()
    if not getattr(lib, "_st_declared", False):
        vp, cp, u64, i64 = C.c_void_p, C.c_char_p, C.c_uint64, C.c_int64
        for name, (res, args) in {
            "mx_st_last_error": (cp, []), "mx_st_open": (vp, [cp]), "mx_st_header": (vp, [vp]), "mx_st_header_len": (u64, [vp]),
            "mx_st_data": (vp, [vp]), "mx_st_data_len": (u64, [vp]), "mx_st_close": (None, [vp]),
            "mx_awq_dequant": (C.c_int, [vp, vp, vp, i64, i64, i64, vp, C.c_int]),
            "mx_gptq_dequant": (C.c_int, [vp, vp, vp, vp, i64, i64, i64, vp, C.c_int]),
        }.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        lib._st_declared = True
    return lib


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        L = self._lib = _lib_st()
        self._h = L.mx_st_open(path.encode())
        if not self._h:
            raise IOError(L.mx_st_last_error().decode())
        hdr = C.string_at(L.mx_st_header(self._h), L.mx_st_header_len(self._h))
        try:
            meta = json.loads(hdr)
        except Exception as e:
            self.close()
            raise IOError(f"safetensors: header of {path} is not JSON: {e}")
        self.metadata = meta.pop("__metadata__", {})
        n = L.mx_st_data_len(self._h)
        self._data = np.ctypeslib.as_array((C.c_uint8 * n).from_address(L.mx_st_data(self._h)))
        self.tensors = {}
        for name, t in meta.items():
            lo, hi = t["data_offsets"]
            if not (0 <= lo <= hi <= n) or t["dtype"] not in _DT:
                self.close()
                raise IOError(f"safetensors: tensor {name} of {path} has bad offsets or dtype {t['dtype']}")
            self.tensors[name] = (t["dtype"], tuple(t["shape"]), lo, hi)

    def numpy(self, name: str) -> np.ndarray:
        """Zero-copy view when the payload is aligned for its dtype, otherwise a copy.  BF16 comes back as uint16 bit patterns."""
        dt, shape, lo, hi = self.tensors[name]
        raw = self._data[lo:hi]
        nd = np.dtype(_DT[dt])
        if raw.ctypes.data % nd.alignment:
            raw = raw.copy()
        return raw.view(nd).reshape(shape)

    def float32(self, name: str) -> np.ndarray:
        dt = self.tensors[name][0]
        a = self.numpy(name)
        if dt == "BF16":
            return (a.astype(np.uint32) << 16).view(np.float32)
        return a.astype(np.float32)

    def close(self):
        if getattr(self, "_h", None):
            self._data = None
            self._lib.mx_st_close(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


class SafetensorsModel:
    """All shards of a checkpoint directory behind one name -> tensor map."""

    def __init__(self, directory: str):
        idx = os.path.join(directory, "model.safetensors.index.json")
        if os.path.exists(idx):
            wm = json.load(open(idx))["weight_map"]
            files = sorted(set(wm.values()))
        else:
            files = sorted(os.path.basename(p) for p in glob.glob(os.path.join(directory, "*.safetensors")))
        if not files:
            raise IOError(f"no .safetensors files in {directory}")
        self.files = [SafetensorsFile(os.path.join(directory, f)) for f in files]
        self.where = {}
        for f in self.files:
            for name in f.tensors:
                self.where[name] = f

    def names(self) -> Iterable[str]:
        return self.where.keys()

    def has(self, name: str) -> bool:
        return name in self.where

    def shape(self, name: str) -> tuple:
        return self.where[name].tensors[name][1]

    def dtype(self, name: str) -> str:
        return self.where[name].tensors[name][0]

    def numpy(self, name: str) -> np.ndarray:
        return self.where[name].numpy(name)

    def float32(self, name: str) -> np.ndarray:
        return self.where[name].float32(name)


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """``tensors``: name -> numpy array, or (dtype string, array) to force e.g. "BF16" for a uint16 array."""
    rev = {np.dtype(v): k for k, v in _DT.items() if k not in ("BOOL", "BF16", "U16")}
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, a in tensors.items():
        dt = None
        if isinstance(a, tuple):
            dt, a = a
        a = np.ascontiguousarray(a)
        dt = dt or rev[a.dtype]
        b = a.tobytes()
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def awq_dequant(qweight: np.ndarray, qzeros: np.ndarray, scales: np.ndarray, group: int, nthreads: int = 8) -> np.ndarray:
    """AWQ gemm-packed linear -> fp32 [out, in]."""
    in_f, out_f = qweight.shape[0], qweight.shape[1] * 8
    qw, qz, sc = (np.ascontiguousarray(qweight, dtype=np.int32), np.ascontiguousarray(qzeros, dtype=np.int32), np.ascontiguousarray(scales, dtype=np.float16))
    if qz.shape != (in_f // group, out_f // 8) or sc.shape != (in_f // group, out_f):
        raise ValueError(f"awq: qzeros {qz.shape} / scales {sc.shape} do not match qweight {qw.shape} with group {group}")
    out = np.empty((out_f, in_f), dtype=np.float32)
    L = _lib_st()
    if L.mx_awq_dequant(qw.ctypes.data, qz.ctypes.data, sc.ctypes.data, in_f, out_f, group, out.ctypes.data, nthreads) != 0:
        raise ValueError(L.mx_st_last_error().decode())
    return out


def gptq_dequant(qweight: np.ndarray, qzeros: np.ndarray, scales: np.ndarray, group: int, g_idx: np.ndarray | None = None, nthreads: int = 8) -> np.ndarray:
    """AutoGPTQ 4-bit linear -> fp32 [out, in]."""
    in_f, out_f = qweight.shape[0] * 8, qweight.shape[1]
    qw, qz, sc = (np.ascontiguousarray(qweight, dtype=np.int32), np.ascontiguousarray(qzeros, dtype=np.int32), np.ascontiguousarray(scales, dtype=np.float16))
    n_groups = sc.shape[0]
    if qz.shape != (n_groups, out_f // 8) or sc.shape[1] != out_f:
        raise ValueError(f"gptq: qzeros {qz.shape} / scales {sc.shape} do not match qweight {qw.shape}")
    gi = None if g_idx is None else np.ascontiguousarray(g_idx, dtype=np.int32)
    if gi is not None and (gi.shape != (in_f,) or gi.min() < 0 or gi.max() >= n_groups):
        raise ValueError("gptq: g_idx out of range")
    if gi is None and (in_f + group - 1) // group > n_groups:
        raise ValueError("gptq: too few groups for in_features / group_size")
    out = np.empty((out_f, in_f), dtype=np.float32)
    L = _lib_st()
    if L.mx_gptq_dequant(qw.ctypes.data, qz.ctypes.data, sc.ctypes.data, None if gi is None else gi.ctypes.data, in_f, out_f, group,
                         out.ctypes.data, nthreads) != 0:
        raise ValueError(L.mx_st_last_error().decode())
    return out
