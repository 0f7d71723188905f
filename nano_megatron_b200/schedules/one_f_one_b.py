"""Non-interleaved 1F1B pipeline schedule.

Signature and semantics of ``forward_backward_1f1b`` follow
nano_megatron/schedules/one_f_one_b.py:41-322: warm-up forwards (``min(p - rank
- 1, M)``), steady one-forward-one-backward, cool-down backwards; each
microbatch loss is scaled by ``1/M`` and the last stage returns their sum; with
a DDP wrapper every backward runs under ``no_sync()`` and one
``finish_grad_sync()`` closes the step.

The exchange order with a neighbour is fixed so that blocking transports cannot
deadlock: towards the next stage "receive gradient, then send activation",
towards the previous stage "send gradient, then receive activation".  The
activation shape comes from the stage (``[mb, S/t, H]`` under sequence
parallelism).
"""
from __future__ import annotations

from collections import deque
from contextlib import nullcontext
from typing import TYPE_CHECKING, Optional

import torch
from torch import Tensor

from ..parallel.context import ParallelContext, is_pipeline_first_stage, is_pipeline_last_stage
from .p2p import drain_pending_sends, recv_backward, recv_forward, send_backward, send_forward

if TYPE_CHECKING:
    from ..distributed.ddp import DistributedDataParallel
    from ..models.pipeline import PipelineStage


def warmup_microbatches(pp_size: int, pp_rank: int, num_microbatches: int) -> int:
    if pp_size < 1:
        raise ValueError(f"pp_size must be >= 1, got {pp_size}")
    if not 0 <= pp_rank < pp_size:
        raise ValueError(f"pp_rank ({pp_rank}) out of range for pp_size={pp_size}")
    if num_microbatches < 1:
        raise ValueError(f"num_microbatches must be >= 1, got {num_microbatches}")
    return min(pp_size - pp_rank - 1, num_microbatches)


def forward_backward_1f1b(*, stage: "PipelineStage", ctx: ParallelContext, input_ids: Tensor, labels: Tensor,
                          positions: Optional[Tensor] = None, num_microbatches: int,
                          ddp: Optional["DistributedDataParallel"] = None) -> Optional[Tensor]:
    if num_microbatches < 1:
        raise ValueError(f"num_microbatches must be >= 1, got {num_microbatches}")
    if input_ids.dim() != 2:
        raise ValueError(f"input_ids must be [B, S], got shape {tuple(input_ids.shape)}")
    batch = input_ids.size(0)
    if batch % num_microbatches != 0:
        raise ValueError(f"input_ids.size(0) ({batch}) must be divisible by num_microbatches ({num_microbatches})")
    if labels.shape != input_ids.shape:
        raise ValueError(f"labels shape {tuple(labels.shape)} must match input_ids shape {tuple(input_ids.shape)}")
    if positions is not None and positions.shape != input_ids.shape:
        raise ValueError(f"positions shape {tuple(positions.shape)} must match input_ids shape "
                         f"{tuple(input_ids.shape)}")
    mb = batch // num_microbatches
    seq_len = input_ids.size(1)
    shape_fn = getattr(stage, "activation_shape", None)
    act_shape = shape_fn(mb, seq_len) if shape_fn is not None else (mb, seq_len, stage.config.hidden_size)
    try:
        first_param = next(stage.parameters())
    except StopIteration as exc:
        raise RuntimeError("pipeline stage has no parameters") from exc
    dtype, device = first_param.dtype, first_param.device

    first, last = is_pipeline_first_stage(ctx), is_pipeline_last_stage(ctx)
    n_warm = warmup_microbatches(ctx.pipeline_parallel_size, ctx.pipeline_parallel_rank, num_microbatches)
    n_steady = num_microbatches - n_warm
    in_flight: deque[tuple[Tensor, Tensor]] = deque()  # (stage input, stage output) awaiting backward
    losses: list[Tensor] = []

    def piece(t: Optional[Tensor], i: int) -> Optional[Tensor]:
        return None if t is None else t[i * mb:(i + 1) * mb]

    def fetch_input(i: int) -> Tensor:
        if first:
            return piece(input_ids, i)
        return recv_forward(ctx, shape=act_shape, dtype=dtype, device=device)

    def run_forward(i: int, x: Tensor) -> Tensor:
        if not first and not x.requires_grad:
            x.requires_grad_(True)  # received activations are leaves; their grad goes upstream
        out = stage(x, positions=piece(positions, i))
        if last:
            out = stage.shifted_cross_entropy(out, piece(labels, i)) / num_microbatches
            losses.append(out)
        return out

    def run_backward(x: Tensor, out: Tensor, grad_out: Optional[Tensor]) -> Optional[Tensor]:
        with (ddp.no_sync() if ddp is not None else nullcontext()):
            if last:
                out.backward()
            else:
                torch.autograd.backward(tensors=out, grad_tensors=grad_out)
        return None if first else x.grad

    def grad_for(out: Tensor) -> Optional[Tensor]:
        return None if last else recv_backward(ctx, shape=tuple(out.shape), dtype=out.dtype, device=out.device)

    # warm-up: forwards only
    for i in range(n_warm):
        x = fetch_input(i)
        out = run_forward(i, x)
        send_forward(ctx, out)
        in_flight.append((x, out))

    # steady state: forward microbatch i, then backward the oldest one in flight
    nxt = fetch_input(n_warm) if n_steady > 0 else None
    for k in range(n_steady):
        i = n_warm + k
        x = nxt
        out = run_forward(i, x)
        grad_out = None
        if not last:
            grad_out = recv_backward(ctx, shape=tuple(out.shape), dtype=out.dtype, device=out.device)
            send_forward(ctx, out)
        in_flight.append((x, out))
        old_x, old_out = in_flight.popleft()
        grad_in = run_backward(old_x, old_out, grad_out)
        if grad_in is not None:
            send_backward(ctx, grad_in)
        nxt = fetch_input(i + 1) if k + 1 < n_steady else None

    # cool-down: drain the remaining backwards
    while in_flight:
        old_x, old_out = in_flight.popleft()
        grad_in = run_backward(old_x, old_out, grad_for(old_out))
        if grad_in is not None:
            send_backward(ctx, grad_in)

    drain_pending_sends()
    if ddp is not None:
        ddp.finish_grad_sync()
    if not last:
        return None
    assert losses, "last stage produced no microbatch losses"
    return torch.stack(losses).sum()
