"""Placement planning: does the checkpoint fit one GPU, and if not over how many should it be sharded.

Same accounting as the reference planner (src/loaders/memory_plan.cpp:56-149): weights = sum of tensor payload bytes,
KV reserve = 2 * kv_heads * ctx * head_dim * bytes over the layers that keep KV (hybrid families: every
``full_attention_interval``-th layer), a flat workspace margin, compared with a safety fraction of device memory.
Differences: the device is a B200 (about 180 GB, probed with ``torch.cuda.mem_get_info`` when a GPU is visible, else
the nominal size), shard counts are powers of two (tensor/expert parallel ranks), the recurrent state of hybrid
models is counted, and ``describe()`` prints the per-GPU share.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .gguf import GGUFReader

B200_BYTES = 183_359 * 1024 * 1024
SAFETY = 0.90
WORKSPACE_BYTES = 3 * 1024 ** 3


@dataclass
class PlacementPlan:
    weights_bytes: int = 0
    kv_bytes: int = 0
    state_bytes: int = 0
    ws_bytes: int = WORKSPACE_BYTES
    per_gpu_bytes: int = 0
    avail_gpus: int = 1
    n_gpus: int = 1
    forced: bool = False
    fits: bool = True
    note: str = ""

    @property
    def need_bytes(self) -> int:
        return self.weights_bytes + self.kv_bytes + self.state_bytes + self.ws_bytes

    def describe(self) -> str:
        gb = lambda b: f"{b / 1e9:.1f} GB"
        share = (self.weights_bytes + self.kv_bytes + self.state_bytes) / max(self.n_gpus, 1) + self.ws_bytes
        return (f"[plan] weights {gb(self.weights_bytes)} + kv {gb(self.kv_bytes)} + state {gb(self.state_bytes)} + workspace {gb(self.ws_bytes)}"
                f" = {gb(self.need_bytes)}; {gb(self.per_gpu_bytes)} usable per GPU, {self.avail_gpus} visible -> {self.n_gpus} GPU(s), "
                f"about {gb(share)} each: {self.note}")


def estimate_kv_bytes(kv: dict, ctx: int, n_seqs: int = 1, bytes_per_elem: int = 2) -> int:
    a = kv.get("general.architecture")
    if a is None:
        return 0
    g = lambda k, d=0: int(kv.get(f"{a}.{k}", d) or d)
    n_layers, n_q = g("block_count"), g("attention.head_count")
    n_kv = kv.get(f"{a}.attention.head_count_kv", n_q)
    n_kv = max(int(v) for v in n_kv) if isinstance(n_kv, list) else int(n_kv or n_q)
    hd = g("attention.key_length") or (g("embedding_length") // n_q if n_q else 0)
    if not (n_layers and n_kv and hd):
        return 0
    interval = g("full_attention_interval", 1)
    n_full = (n_layers + interval - 1) // interval if interval > 1 else n_layers
    return 2 * n_full * n_kv * hd * ctx * bytes_per_elem * n_seqs


def estimate_state_bytes(kv: dict, n_seqs: int = 1) -> int:
    a = kv.get("general.architecture")
    g = lambda k, d=0: int(kv.get(f"{a}.{k}", d) or d)
    interval = g("full_attention_interval", 0)
    if interval <= 1:
        return 0
    n_layers, n_v, n_k, d = g("block_count"), g("ssm.time_step_rank"), g("ssm.group_count"), g("ssm.state_size")
    n_lin = n_layers - n_layers // interval
    conv = (g("ssm.conv_kernel", 4) - 1) * (2 * n_k + n_v) * d * 2
    return n_seqs * n_lin * (n_v * d * d * 4 + conv)


def visible_gpus() -> tuple:
    """(count, usable bytes per GPU)."""
    try:
        import torch
        if torch.cuda.is_available():
            n = torch.cuda.device_count()
            _, total = torch.cuda.mem_get_info(0)
            return n, int(total * SAFETY)
    except Exception:
        pass
    return 1, int(B200_BYTES * SAFETY)


def plan_placement(path_or_reader, n_gpus: int = 0, ctx: int = 8192, n_seqs: int = 1, avail: Optional[int] = None,
                   per_gpu_bytes: Optional[int] = None) -> PlacementPlan:
    """``n_gpus`` 0 = decide; otherwise the request is respected (clamped to the visible GPUs)."""
    r = path_or_reader if isinstance(path_or_reader, GGUFReader) else GGUFReader(path_or_reader)
    p = PlacementPlan()
    p.weights_bytes = r.total_tensor_bytes
    p.kv_bytes = estimate_kv_bytes(r.kv, ctx, n_seqs)
    p.state_bytes = estimate_state_bytes(r.kv, n_seqs)
    n_vis, usable = visible_gpus()
    p.avail_gpus = avail if avail is not None else n_vis
    p.per_gpu_bytes = per_gpu_bytes if per_gpu_bytes is not None else usable
    if n_gpus > 0:
        p.forced = True
        p.n_gpus = min(n_gpus, max(p.avail_gpus, 1))
        p.fits = (p.weights_bytes + p.kv_bytes + p.state_bytes) / p.n_gpus + p.ws_bytes <= p.per_gpu_bytes
        p.note = f"forced --gpus {n_gpus} (using {p.n_gpus})" + ("" if p.fits else " -- does not fit, expect an out-of-memory error")
        return p
    if p.need_bytes <= p.per_gpu_bytes:
        p.n_gpus, p.note = 1, "fits one GPU"
        return p
    n = 2
    while n < p.avail_gpus and (p.weights_bytes + p.kv_bytes + p.state_bytes) / n + p.ws_bytes > p.per_gpu_bytes:
        n *= 2
    if p.avail_gpus >= 2:
        p.n_gpus = min(n, p.avail_gpus)
        p.fits = (p.weights_bytes + p.kv_bytes + p.state_bytes) / p.n_gpus + p.ws_bytes <= p.per_gpu_bytes
        p.note = f"over one GPU -> tensor/expert parallel over {p.n_gpus}" + ("" if p.fits else " (still tight: may run out of memory)")
        return p
    p.n_gpus, p.fits, p.note = 1, False, "over one GPU but only one is visible (may run out of memory)"
    return p
