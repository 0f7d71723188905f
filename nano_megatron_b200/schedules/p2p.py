"""Pipeline point-to-point helpers over ``ctx.backend`` (NCCL p2p on GPUs).

Same four functions as nano_megatron/schedules/p2p.py:29-92: receives return
``None`` and sends are no-ops at the pipeline ends.  When the backend offers
``isend`` the sends do not make the compute stream wait for the peer: the work
handle is parked in :data:`_PENDING_SENDS` and :func:`drain_pending_sends`
(called by the schedule at the end of a step) waits for them.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
from torch import Tensor

from ..parallel.context import (
    ParallelContext,
    is_pipeline_first_stage,
    is_pipeline_last_stage,
    pipeline_next_rank,
    pipeline_prev_rank,
)

_PENDING_SENDS: list[tuple[Any, Tensor]] = []


def _send(ctx: ParallelContext, tensor: Tensor, dst: int) -> None:
    isend = getattr(ctx.backend, "isend", None)
    if isend is not None:
        _PENDING_SENDS.append((isend(tensor, dst=dst, group=ctx.pipeline_parallel_group), tensor))
    else:
        ctx.backend.send(tensor, dst=dst, group=ctx.pipeline_parallel_group)


def drain_pending_sends() -> None:
    while _PENDING_SENDS:
        work, _tensor = _PENDING_SENDS.pop(0)
        if hasattr(work, "wait"):
            work.wait()


def recv_forward(ctx: ParallelContext, *, shape: tuple[int, ...], dtype: torch.dtype,
                 device: torch.device) -> Optional[Tensor]:
    src = None if is_pipeline_first_stage(ctx) else pipeline_prev_rank(ctx)
    if src is None:
        return None
    return ctx.backend.recv(torch.empty(shape, dtype=dtype, device=device), src=src,
                            group=ctx.pipeline_parallel_group)


def send_forward(ctx: ParallelContext, tensor: Tensor) -> None:
    dst = None if is_pipeline_last_stage(ctx) else pipeline_next_rank(ctx)
    if dst is not None:
        _send(ctx, tensor, dst)


def recv_backward(ctx: ParallelContext, *, shape: tuple[int, ...], dtype: torch.dtype,
                  device: torch.device) -> Optional[Tensor]:
    src = None if is_pipeline_last_stage(ctx) else pipeline_next_rank(ctx)
    if src is None:
        return None
    return ctx.backend.recv(torch.empty(shape, dtype=dtype, device=device), src=src,
                            group=ctx.pipeline_parallel_group)


def send_backward(ctx: ParallelContext, tensor: Tensor) -> None:
    dst = None if is_pipeline_first_stage(ctx) else pipeline_prev_rank(ctx)
    if dst is not None:
        _send(ctx, tensor, dst)
