"""Expert banks that do not fit the GPU: kept in host memory, copied into a shared device buffer before their layer runs.

A budget (bytes of expert weights per device) is set before the graph is built.  Layers are admitted in order; once the budget is
used up, the expert banks of the remaining MoE layers stay in page-locked host memory, and each of those layers copies its banks
into one staging area on the device (shared by all spilled layers, sized for the largest) at the start of its forward.  The copies
are ordinary stream-ordered host-to-device copies, so they may sit inside CUDA graphs, and the kernels only ever see device memory.
A spilled layer costs its bank size over PCIe per forward: the point is that a model whose experts exceed the memory still runs,
and that the resident part keeps its speed.

Reference parity: src/model/gptoss_tp.cpp:59-68,390-403 (per-card budget; expert planes past it are allocated in host memory and
read by the kernels over PCIe).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..ops.weights import QuantWeight


class ExpertSpill:
    def __init__(self, budget_bytes: int):
        self.budget = int(budget_bytes)
        self.resident_bytes = 0
        self.spilled_bytes = 0
        self.layers_spilled = 0
        self._stage: dict = {}            # (slot, plane) -> uint8 device buffer

    def admit(self, nbytes: int) -> bool:
        """True: the bank stays on the device (and counts against the budget)."""
        if self.resident_bytes + nbytes <= self.budget:
            self.resident_bytes += nbytes
            return True
        self.spilled_bytes += nbytes
        self.layers_spilled += 1
        return False

    def to_host(self, slot: int, w: QuantWeight) -> QuantWeight:
        """The bank with its planes in host memory (page-locked when it came from a GPU); reserves the staging area for it."""
        dev = w.device
        planes = []
        for i, t in enumerate(w.planes()):
            if t is None:
                planes.append(None)
                continue
            nbytes = t.numel() * t.element_size()
            buf = self._stage.get((slot, i))
            if buf is None or buf.numel() < nbytes or buf.device != dev:
                self._stage[(slot, i)] = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            h = t.detach().to("cpu").contiguous()
            if dev.type == "cuda":
                h = h.pin_memory()
            planes.append(h)
        out = QuantWeight(w.fmt, w.N, w.K, w.E, *planes, dual=w.dual)
        out._home = dev
        return out

    def fetch(self, slot: int, host: QuantWeight) -> QuantWeight:
        """The bank on the device, inside the staging area (valid until the next fetch into the same slot)."""
        planes = []
        for i, t in enumerate(host.planes()):
            if t is None:
                planes.append(None)
                continue
            nbytes = t.numel() * t.element_size()
            view = self._stage[(slot, i)][:nbytes].view(t.dtype).reshape(t.shape)
            view.copy_(t, non_blocking=True)
            planes.append(view)
        return QuantWeight(host.fmt, host.N, host.K, host.E, *planes, dual=host.dual)


_active: list[Optional[ExpertSpill]] = [None]


def configure(budget_gb: Optional[float]) -> Optional[ExpertSpill]:
    """Sets the expert budget for the graphs built from now on (None: no limit, nothing spills).  Returns the accounting object."""
    _active[0] = None if budget_gb is None else ExpertSpill(int(float(budget_gb) * 1e9))
    return _active[0]


def active() -> Optional[ExpertSpill]:
    if _active[0] is None and os.environ.get("MX_EXPERT_BUDGET_GB"):
        configure(float(os.environ["MX_EXPERT_BUDGET_GB"]))
    return _active[0]
