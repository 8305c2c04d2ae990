"""ctypes access to the two native libraries.

``host()`` is the C++ host library (GGUF, codecs, tokenizer, packing); it is built on first use
when a compiler is present.  ``cuda()`` is the sm_100a kernel library; it is *never* silently
replaced: on a machine with a GPU a missing or unloadable kernel library raises.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

from . import _build

_lock = threading.Lock()
_host = None
_cuda = None


class NativeError(RuntimeError):
    pass


def host() -> C.CDLL:
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                path = _build.build_host()
                lib = C.CDLL(str(path))
                _declare_host(lib)
                _host = lib
    return _host


def cuda() -> C.CDLL:
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                path = _build.CUDA_LIB
                if not path.exists():
                    path = _build.build_cuda()
                try:
                    lib = C.CDLL(str(path))
                except OSError as e:  # pragma: no cover - needs a broken install
                    raise NativeError(f"cannot load the sm_100a kernel library {path}: {e}") from e
                _cuda = lib
    return _cuda


def cuda_loaded_path() -> Path | None:
    return _build.CUDA_LIB if _cuda is not None else None


def host_error() -> str:
    return host().mx_last_error().decode("utf-8", "replace")


def _declare_host(lib: C.CDLL) -> None:
    vp, cp, u64, i32, i64 = C.c_void_p, C.c_char_p, C.c_uint64, C.c_int32, C.c_int64
    sig = {
        "mx_last_error": (cp, []),
        "mx_gguf_open": (vp, [cp]),
        "mx_gguf_meta_json": (vp, [vp]),
        "mx_gguf_meta_json_len": (u64, [vp]),
        "mx_gguf_tensor_ptr": (vp, [vp, i64]),
        "mx_gguf_close": (None, [vp]),
        "mx_ggufw_new": (vp, []),
        "mx_ggufw_free": (None, [vp]),
        "mx_ggufw_kv_u32": (None, [vp, cp, C.c_uint32]),
        "mx_ggufw_kv_i32": (None, [vp, cp, i32]),
        "mx_ggufw_kv_u64": (None, [vp, cp, u64]),
        "mx_ggufw_kv_f32": (None, [vp, cp, C.c_float]),
        "mx_ggufw_kv_bool": (None, [vp, cp, C.c_int]),
        "mx_ggufw_kv_str": (None, [vp, cp, cp, u64]),
        "mx_ggufw_kv_arr_str": (None, [vp, cp, cp, vp, u64]),
        "mx_ggufw_kv_arr_i32": (None, [vp, cp, vp, u64]),
        "mx_ggufw_kv_arr_f32": (None, [vp, cp, vp, u64]),
        "mx_ggufw_add_tensor": (u64, [vp, cp, C.c_int, vp, i32]),
        "mx_ggufw_begin": (C.c_int, [vp, cp]),
        "mx_ggufw_write": (C.c_int, [vp, vp, u64]),
        "mx_ggufw_end": (C.c_int, [vp]),
        "mx_dequantize": (C.c_int, [i32, vp, vp, u64]),
        "mx_quantize": (C.c_int, [i32, vp, vp, u64, u64, C.c_int]),
        "mx_bytes_for": (u64, [i32, u64]),
        "mx_type_block_elems": (C.c_int, [i32]),
        "mx_type_block_bytes": (C.c_int, [i32]),
        "mx_type_name": (cp, [i32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    # optional groups are declared by the modules that own them (tokenizer, packing, ...)
