"""Block codecs: numpy faces over the C++ encoders/decoders (``csrc/host/quant.cpp``).

Reference parity: include/ie/dequant_ref.hpp (decode), include/ie/quantize.hpp (encode).
"""
from __future__ import annotations

import os

import numpy as np

from .. import _lib


def dequantize(raw: np.ndarray, ttype: int, n_elements: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
    out = np.empty(n_elements, dtype=np.float32)
    rc = _lib.host().mx_dequantize(int(ttype), raw.ctypes.data, out.ctypes.data, n_elements)
    if rc != 0:
        raise ValueError(f"cannot dequantize ggml type {ttype} ({n_elements} elements)")
    return out


def quantize(x: np.ndarray, ttype: int, nthreads: int | None = None) -> np.ndarray:
    """Quantise a 2-D (rows, cols) float array row by row; returns the packed bytes."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim == 1:
        x = x[None, :]
    rows = int(np.prod(x.shape[:-1]))
    cols = x.shape[-1]
    lib = _lib.host()
    nb = lib.mx_bytes_for(int(ttype), rows * cols)
    if nb == 0 or cols % lib.mx_type_block_elems(int(ttype)):
        raise ValueError(f"row length {cols} is not a whole number of blocks of ggml type {ttype}")
    out = np.empty(nb, dtype=np.uint8)
    rc = lib.mx_quantize(int(ttype), x.ctypes.data, out.ctypes.data, rows, cols, nthreads or min(16, os.cpu_count() or 1))
    if rc != 0:
        raise ValueError(f"cannot quantize to ggml type {ttype}")
    return out


def set_kquant_fit(mode: int) -> None:
    """Q4_K / Q5_K sub-block fit of :func:`quantize`: 0 = per sub-block the better of the two fits below (default), 1 = alternating
    least squares, 2 = the importance-weighted grid search of ggml's K-quant encoders."""
    _lib.host().mx_quantize_set_kquant_fit(int(mode))
