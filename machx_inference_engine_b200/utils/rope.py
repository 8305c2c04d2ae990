"""Rotary tables.  All RoPE flavours the models need are baked into (cos, sin) tables indexed by
position, so the device kernel is a table lookup: plain NEOX frequencies, llama-3 frequency
factors (``rope_freqs.weight``) and YaRN (ggml's formula: corrected dims, ramp mix, mscale on
cos/sin).  Reference parity: src/ops/elementwise.cpp:595-786 (rope / rope_ff / rope_yarn).
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def _yarn_corr_dim(n_dims: int, n_ctx_orig: int, n_rot: float, base: float) -> float:
    return n_dims * math.log(n_ctx_orig / (n_rot * 2 * math.pi)) / (2 * math.log(base))


def rope_tables(max_pos: int, n_rot: int, theta: float, freq_factors: Optional[torch.Tensor] = None, scaling_type: str = "none",
                scaling_factor: float = 1.0, orig_ctx: int = 0, beta_fast: float = 32.0, beta_slow: float = 1.0,
                device="cpu") -> tuple[torch.Tensor, torch.Tensor]:
    """Returns fp32 (cos, sin), each [max_pos, n_rot/2]."""
    half = n_rot // 2
    i0 = torch.arange(0, n_rot, 2, dtype=torch.float64)
    inv = theta ** (-i0 / n_rot)
    if freq_factors is not None:
        inv = inv / freq_factors.to(torch.float64).cpu()[:half]
    pos = torch.arange(max_pos, dtype=torch.float64).unsqueeze(1)
    extrap = pos * inv.unsqueeze(0)
    mscale = 1.0
    if scaling_type == "yarn" and scaling_factor > 1.0 and orig_ctx > 0:
        freq_scale = 1.0 / scaling_factor
        lo = max(0.0, math.floor(_yarn_corr_dim(n_rot, orig_ctx, beta_fast, theta)))
        hi = min(n_rot - 1.0, math.ceil(_yarn_corr_dim(n_rot, orig_ctx, beta_slow, theta)))
        ramp = 1.0 - ((i0 / 2 - lo) / max(0.001, hi - lo)).clamp(0.0, 1.0)        # ext_factor = 1
        ang = freq_scale * extrap * (1.0 - ramp) + extrap * ramp
        mscale = 1.0 + 0.1 * math.log(1.0 / freq_scale)
    elif scaling_type == "linear" and scaling_factor > 1.0:
        ang = extrap / scaling_factor
    else:
        ang = extrap
    return (torch.cos(ang) * mscale).to(torch.float32).to(device).contiguous(), (torch.sin(ang) * mscale).to(torch.float32).to(device).contiguous()
