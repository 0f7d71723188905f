"""Opt-in NVTX ranges around the phases of a step and the fused paths.

The reference has no tracing at all (its benchmark scripts bracket
``time.perf_counter()`` with ``torch.cuda.synchronize()``,
``scripts/benchmark_dp.py:111-134``).  Here ``NMB_NVTX=1`` (or
:func:`enable`) turns the ranges on; when off, ``nvtx_range`` costs one
attribute read.  Ranges are host-side markers: inside a captured CUDA graph
they are only emitted while the graph is being captured, so trace an eager
run (``Trainer(..., use_cuda_graph=False)``) to see them per step.
"""
from __future__ import annotations

import contextlib
import os
from typing import Iterator

import torch

_enabled = os.environ.get("NMB_NVTX", "0") not in ("", "0")


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


@contextlib.contextmanager
def nvtx_range(name: str) -> Iterator[None]:
    if not _enabled or not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
