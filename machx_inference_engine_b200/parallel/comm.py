"""Process-group plumbing and the *baseline* collectives (plain NCCL / gloo).

One process per GPU; ``torch.distributed`` carries the control plane and the baseline data plane.
The product data plane -- GEMM fused with all-reduce over NVLink peer memory -- lives in
``parallel/fused.py`` and is selected through :class:`ParallelCtx.fused`.

Reference parity: ``DeviceFleet`` (include/ie/allocator.hpp:51-92, src/core/allocator.cpp:96-193):
``copy_across`` -> broadcast / send-recv, ``all_reduce_sum_fp16`` -> all_reduce.  The reference sums
on the host in fixed device order; NCCL's order is fixed for a given communicator and size, and the
fused kernels sum in rank order, so results are run-to-run deterministic here as well.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelCtx:
    rank: int = 0
    world: int = 1
    group: Optional[object] = None
    fused: Optional[object] = None          # parallel.fused.FusedComm when the peer-memory path is on
    sharded: Optional[object] = None        # parallel.sharded.ShardedComm: row-sharded prefill (needs `fused` for its reduce-scatter)
    mode: str = "tp"                        # "tp": tensor/expert parallel, "pp": layer split
    _ctrl: Optional[object] = None          # gloo group for host-side control messages (step plans)

    @property
    def enabled(self) -> bool:
        return self.world > 1

    # ---- baseline collectives ------------------------------------------------------------
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        if t.device.type == "cpu" and t.dtype == torch.bfloat16:
            f = t.to(torch.float32)
            dist.all_reduce(f, group=self.group)
            t.copy_(f)
            return t
        dist.all_reduce(t, group=self.group)
        return t

    def all_gather_cols(self, t: torch.Tensor) -> torch.Tensor:
        """[R, C_local] on every rank -> [R, C_local * world] (rank-major columns)."""
        if self.world == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world > 1:
            dist.broadcast(t, src=src, group=self.group)
        return t

    def barrier(self) -> None:
        if self.world > 1:
            dist.barrier(group=self.group)

    def control_group(self):
        """A gloo group over the same ranks: control-plane objects travel over TCP on the host, so ranks that wait for
        the next step plan block in a socket read instead of spinning a GPU."""
        if self.world == 1:
            return None
        if self._ctrl is None:
            self._ctrl = dist.new_group(backend="gloo") if dist.get_backend() != "gloo" else (self.group or dist.group.WORLD)
        return self._ctrl

    def broadcast_object(self, obj, src: int = 0):
        if self.world == 1:
            return obj
        box = [obj if self.rank == src else None]
        dist.broadcast_object_list(box, src=src, group=self.control_group())
        return box[0]

    def send(self, t: torch.Tensor, dst: int) -> None:
        dist.send(t, dst=dst, group=self.group)

    def recv(self, t: torch.Tensor, src: int) -> torch.Tensor:
        dist.recv(t, src=src, group=self.group)
        return t

    def shard(self, n: int) -> tuple[int, int]:
        """Even [lo, hi) share of n items for this rank (n must divide)."""
        if n % self.world:
            raise ValueError(f"{n} is not divisible by the parallel size {self.world}")
        per = n // self.world
        return self.rank * per, (self.rank + 1) * per


def init_from_env(device_type: str = "cuda", timeout_s: int = 600) -> ParallelCtx:
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (torchrun contract)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world == 1:
        return ParallelCtx()
    if not dist.is_initialized():
        import datetime
        backend = "nccl" if device_type == "cuda" else "gloo"
        if device_type == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group(backend=backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
    # MX_PARALLEL=pp selects the layer split (pipeline) instead of tensor/expert parallelism
    mode = "pp" if os.environ.get("MX_PARALLEL", "tp").lower() == "pp" else "tp"
    return ParallelCtx(rank=rank, world=world, group=dist.group.WORLD, mode=mode)
