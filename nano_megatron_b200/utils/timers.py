"""Device-side timing: CUDA events on the launching stream, reduced as the
maximum over ranks.  The reference times with host ``perf_counter`` around
``cuda.synchronize`` (scripts/benchmark_dp.py:111-134); multi-GPU numbers here
are device times, max over ranks."""
from __future__ import annotations

import time
from contextlib import contextmanager
from typing import Any, Callable, Iterator, Optional

import torch


class DeviceTimer:
    """Accumulates named regions; ``summary()`` returns milliseconds per name."""

    def __init__(self, device: Optional[torch.device] = None) -> None:
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self._open: dict[str, Any] = {}
        self._pairs: dict[str, list[tuple[Any, Any]]] = {}
        self._host_ms: dict[str, float] = {}

    @contextmanager
    def region(self, name: str) -> Iterator[None]:
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                self._pairs.setdefault(name, []).append((a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._host_ms[name] = self._host_ms.get(name, 0.0) + (time.perf_counter() - t0) * 1e3

    def summary(self, *, group: Any = None, reduce_max: bool = True) -> dict[str, float]:
        out = dict(self._host_ms)
        if self.cuda:
            torch.cuda.synchronize()
            for name, pairs in self._pairs.items():
                out[name] = sum(a.elapsed_time(b) for a, b in pairs)
        if reduce_max and torch.distributed.is_available() and torch.distributed.is_initialized():
            names = sorted(out)
            t = torch.tensor([out[n] for n in names], dtype=torch.float64,
                             device="cuda" if self.cuda else "cpu")
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX, group=group)
            out = {n: float(v) for n, v in zip(names, t.tolist())}
        return out

    def reset(self) -> None:
        self._pairs.clear()
        self._host_ms.clear()


def time_steps(step: Callable[[], Any], *, warmup: int, steps: int, barrier: Optional[Callable[[], None]] = None) -> float:
    """Milliseconds for ``steps`` calls after ``warmup`` untimed ones (device time on CUDA)."""
    for _ in range(warmup):
        step()
    if barrier is not None:
        barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    return (time.perf_counter() - t0) * 1e3
