"""EXL3 (QTIP-style trellis quantisation, exllamav3) on the host.

A quantised linear layer is three tensors: ``trellis`` int16 [K/16, N/16, 16*bits] (one cyclic bit stream of
``256 * bits`` bits per 16 x 16 tile of the rotated weight), ``suh`` fp16 [K] and ``svh`` fp16 [N]
(sign-and-scale of every input / output feature).  The layer computes

    y = had128(had128(x * suh) @ W_rot) * svh

where ``W_rot`` [K, N] is the decoded trellis and ``had128`` the block-diagonal, normalised 128-point Sylvester
Hadamard transform, so K and N are multiples of 128.  Only the default codebook (no ``mcg`` / ``mul1`` tensors)
is handled.  In GGUF files the trellis is stored verbatim as tensor type 37 with dims {16*bits, N/16, K/16} next
to ``<name>.suh`` / ``<name>.svh`` F16 vectors.

This module holds the decoders (the C++ one of ``csrc/host/exl3.cpp`` and an independent numpy one used as its
oracle in the tests), the dense "effective weight" of a layer, and a generator of random layers (any bit stream is a
valid trellis, which is what the synthetic checkpoints use).

Reference parity: include/ie/exl3.hpp:21-36, src/core/exl3_decode.cpp, src/ops/hadamard.cpp:36,
src/loaders/hf_import.cpp:440-592, tools/exl3/make_oracle.py.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from .. import _lib

GGML_TYPE_EXL3 = 37
HAD = 128
# standard deviation of the codebook over uniformly drawn 16-bit windows (mean is ~0)
CODEBOOK_STD = 1.2437109


def _host():
    lib = _lib.host()
    if not getattr(lib, "_exl3_declared", False):
        lib.mx_exl3_decode.restype = C.c_int
        lib.mx_exl3_decode.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_int, C.c_int]
        lib.mx_hadamard128.restype = C.c_int
        lib.mx_hadamard128.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64]
        lib._exl3_declared = True
    return lib


def trellis_bits(trellis) -> int:
    w = int(trellis.shape[-1])
    if w % 16 or not 1 <= w // 16 <= 8:
        raise ValueError(f"EXL3 trellis rows hold 16 * bits words, bits 1..8 (got {w})")
    return w // 16


def decode_trellis(trellis: torch.Tensor, transpose: bool = False) -> torch.Tensor:
    """int16 [K/16, N/16, 16*bits] -> W_rot fp32 [K, N] (or [N, K])."""
    t = trellis.detach().cpu().contiguous()
    assert t.dtype == torch.int16 and t.dim() == 3
    tk, tn, bits = int(t.shape[0]), int(t.shape[1]), trellis_bits(t)
    out = torch.empty((tn * 16, tk * 16) if transpose else (tk * 16, tn * 16), dtype=torch.float32)
    rc = _host().mx_exl3_decode(t.data_ptr(), tk, tn, bits, out.data_ptr(), int(transpose), 0)
    if rc:
        raise RuntimeError(f"mx_exl3_decode failed ({rc})")
    return out


def code_value_numpy(code: np.ndarray) -> np.ndarray:
    """The procedural codebook: 16-bit window -> weight (fp32 holding an fp16 value)."""
    x = (code.astype(np.uint64) * 89226354 + 64248484) & 0xFFFFFFFF
    x = ((x & 0x8FFF8FFF) ^ 0x3B603B60).astype(np.uint32)
    lo = (x & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32)
    hi = (x >> 16).astype(np.uint16).view(np.float16).astype(np.float32)
    return (lo + hi).astype(np.float16).astype(np.float32)


def decode_trellis_numpy(trellis: np.ndarray) -> np.ndarray:
    """Bit-level decoder written from the format description, independent of the C++ one: the tile's stream is expanded to
    single bits (most significant bit of each 32-bit word first), every weight reads its 16-bit window with cyclic indexing."""
    t = np.ascontiguousarray(trellis).view(np.uint16)
    tk, tn, w16 = t.shape
    bits = w16 // 16
    nb = bits * 256
    words = t[..., 0::2].astype(np.uint32) | (t[..., 1::2].astype(np.uint32) << 16)               # [tk, tn, 8*bits]
    stream = ((words[..., None] >> np.arange(31, -1, -1, dtype=np.uint32)) & 1).reshape(tk, tn, nb).astype(np.uint32)
    tt = np.arange(256)
    idx = (((tt + 1) * bits - 16)[:, None] + np.arange(16)[None, :]) % nb                         # [256, 16] bit positions
    code = (stream[:, :, idx] << np.arange(15, -1, -1, dtype=np.uint32)).sum(-1)                  # [tk, tn, 256]
    vals = code_value_numpy(code)
    # fragment order -> row-major: lane l = t // 8 holds rows {2 (l % 4), +1, +8, +9} of columns {l // 4, l // 4 + 8}
    lane, j = tt // 8, tt % 8
    row = (lane % 4) * 2 + (j % 2) + ((j // 2) % 2) * 8
    col = lane // 4 + (j // 4) * 8
    tile = np.empty((tk, tn, 16, 16), np.float32)
    tile[:, :, row, col] = vals
    return tile.transpose(0, 2, 1, 3).reshape(tk * 16, tn * 16)


def hadamard128(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Normalised Sylvester Hadamard transform of every aligned run of 128 elements along ``dim`` (its own inverse)."""
    x = x.transpose(dim, -1)
    shp = x.shape
    if shp[-1] % HAD:
        raise ValueError("hadamard128 needs a multiple of 128 elements")
    v = x.reshape(-1, HAD).to(torch.float32)
    ln = 1
    while ln < HAD:
        v = v.reshape(-1, HAD // (2 * ln), 2, ln)
        a, b = v[:, :, 0], v[:, :, 1]
        v = torch.stack([a + b, a - b], dim=2)
        ln *= 2
    v = v.reshape(shp) * (1.0 / math.sqrt(HAD))
    return v.transpose(dim, -1)


def effective_weight(trellis: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor) -> torch.Tensor:
    """The dense matrix W [N, K] with y = x W^T equal to the layer's three steps."""
    w = decode_trellis(trellis)                                   # [K, N]
    w = hadamard128(hadamard128(w, dim=0), dim=1)
    w = w * suh.detach().cpu().to(torch.float32).reshape(-1, 1) * svh.detach().cpu().to(torch.float32).reshape(1, -1)
    return w.t().contiguous()


def random_layer(N: int, K: int, bits: int, gen: torch.Generator, std: float = 0.02):
    """A random EXL3 layer whose effective weight has about the given standard deviation: uniform trellis bits decode to the
    codebook's distribution, the Hadamard transforms keep the variance, ``svh`` carries the scale and both vectors random signs."""
    if N % HAD or K % HAD:
        raise ValueError("EXL3 layers need in and out features that are multiples of 128")
    dev = gen.device
    trellis = torch.randint(-32768, 32768, (K // 16, N // 16, 16 * bits), generator=gen, device=dev, dtype=torch.int32).to(torch.int16)
    sg = lambda n: (torch.randint(0, 2, (n,), generator=gen, device=dev) * 2 - 1).to(torch.float32)
    suh = (sg(K) * (1.0 + 0.1 * torch.rand(K, generator=gen, device=dev))).to(torch.float16)
    svh = (sg(N) * (std / CODEBOOK_STD)).to(torch.float16)
    return trellis, suh, svh
