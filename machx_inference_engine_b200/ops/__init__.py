"""Operator entry points used by the model graphs.

Tensors on a CUDA device go to the hand-written sm_100a kernels (``ops.cuda``); tensors on the
CPU go to the fp32 PyTorch oracle (``ops.ref``), which is also what the GPU tests compare with.
There is exactly one GPU implementation per op -- no backend selection, no eager fallback on GPU.
"""
from __future__ import annotations

import functools

from . import ref
from .ref import ACT_GEGLU, ACT_NONE, ACT_SWIGLU, ACT_SWIGLU_OAI, MOE_TILE, MoePacking, moe_max_rows
from .weights import QuantWeight, WFormat, from_dense, from_exl3, from_ggml
from ..utils.profiler import profiler as _prof

_NAMES = [
    "embed", "rmsnorm", "glu", "sigmoid_mul", "scaled_add", "gated_rmsnorm", "qkv_post", "linear", "grouped_linear", "expert_gemv", "expert_group_gemv",
    "attention", "gated_rmsnorm_heads", "conv1d_silu", "deltanet_scan", "moe_route", "moe_pack", "moe_gather", "moe_combine", "argmax", "rep_penalty", "sample",
    "hadamard128",
]


_BACKEND = ["auto"]


def set_backend(name: str) -> None:
    """"auto": CUDA tensors run the engine's kernels, CPU tensors the PyTorch oracle.  "torch": every op runs the PyTorch
    restatement wherever its tensors live -- on a GPU that is cuBLAS / ATen kernels only, the library baseline the benchmarks
    compare the engine's own kernels with."""
    if name not in ("auto", "torch"):
        raise ValueError(name)
    _BACKEND[0] = name


def backend() -> str:
    return _BACKEND[0]


def _first_tensor(args, kwargs):
    import torch
    for a in list(args) + list(kwargs.values()):
        if isinstance(a, torch.Tensor):
            return a
        if isinstance(a, QuantWeight):
            return a.p0
        if isinstance(a, MoePacking):
            return a.packed_token
    raise TypeError("op called without a tensor argument")


def _make(name):
    ref_fn = getattr(ref, name)

    @functools.wraps(ref_fn)
    def op(*args, **kwargs):
        if _BACKEND[0] == "auto" and _first_tensor(args, kwargs).is_cuda:
            from . import cuda
            fn = getattr(cuda, name)
            if _prof.enabled:
                tag = name
                if name == "linear":
                    tag = "gemv" if args[0].shape[0] <= cuda.GEMV_MAX_M else "gemm"
                return _prof.record(tag, fn, args, kwargs)
            return fn(*args, **kwargs)
        if _prof.enabled:
            return _prof.record_host(name, ref_fn, args, kwargs)
        return ref_fn(*args, **kwargs)

    return op


for _n in _NAMES:
    globals()[_n] = _make(_n)

__all__ = _NAMES + ["set_backend", "QuantWeight", "WFormat", "from_dense", "from_exl3", "from_ggml", "MoePacking", "moe_max_rows", "ACT_NONE", "ACT_SWIGLU",
                    "ACT_SWIGLU_OAI", "ACT_GEGLU", "MOE_TILE"]
