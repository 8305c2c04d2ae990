"""Per-op device-time profiler: CUDA events around every op launch, aggregated by op name.

Reference parity: include/ie/kernel_profiler.hpp:23-87 (``ie::ps`` wraps every submit, ``harvest``
sums device time per name) and its front ends ``ie-bench --kprofile*``.  Off by default; when off
the only cost is one attribute test per op call.
"""
from __future__ import annotations

from collections import defaultdict
from contextlib import contextmanager


class KernelProfiler:
    def __init__(self):
        self.enabled = False
        self._pending = []

    def start(self):
        self._pending = []
        self.enabled = True

    def stop(self):
        self.enabled = False

    def record(self, name, fn, args, kwargs):
        import torch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn(*args, **kwargs)
        e1.record()
        self._pending.append((name, e0, e1))
        return out

    def record_host(self, name, fn, args, kwargs):
        """CPU path: wall-clock time of the op (the PyTorch restatement runs synchronously)."""
        import time
        t0 = time.perf_counter()
        out = fn(*args, **kwargs)
        self._pending.append((name, (time.perf_counter() - t0) * 1e3, None))
        return out

    def harvest_ordered(self) -> list:
        """[(name, ms)] in dispatch order; synchronises the device."""
        import torch
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        out = [(name, a if b is None else a.elapsed_time(b)) for name, a, b in self._pending]
        self._pending = []
        return out

    def harvest(self) -> dict:
        """{name: (calls, total_ms)} sorted by total time; synchronises the device."""
        agg = defaultdict(lambda: [0, 0.0])
        for name, ms in self.harvest_ordered():
            agg[name][0] += 1
            agg[name][1] += ms
        return dict(sorted(((k, (v[0], v[1])) for k, v in agg.items()), key=lambda kv: -kv[1][1]))

    @staticmethod
    def format(table: dict) -> str:
        total = sum(v[1] for v in table.values()) or 1.0
        lines = [f"{'op':<24}{'calls':>8}{'total ms':>12}{'avg us':>12}{'share':>8}"]
        for k, (n, ms) in table.items():
            lines.append(f"{k:<24}{n:>8}{ms:>12.3f}{ms / n * 1e3:>12.1f}{ms / total * 100:>7.1f}%")
        lines.append(f"{'TOTAL':<24}{sum(v[0] for v in table.values()):>8}{total:>12.3f}")
        return "\n".join(lines)


profiler = KernelProfiler()


@contextmanager
def profiled():
    profiler.start()
    try:
        yield profiler
    finally:
        profiler.stop()
