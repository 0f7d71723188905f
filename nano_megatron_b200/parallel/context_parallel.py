"""Context-parallel sequence operators (contiguous shards) and the shifted
causal mask; API of nano_megatron/parallel/context_parallel.py:23-273."""
from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from ..distributed.backend import CommBackend


def local_sequence_range(cp_rank: int, cp_size: int, seq_len: int) -> tuple[int, int]:
    if cp_size < 1:
        raise ValueError(f"cp_size must be >= 1, got {cp_size}")
    if not 0 <= cp_rank < cp_size:
        raise ValueError(f"cp_rank must be in [0, {cp_size}), got {cp_rank}")
    if seq_len % cp_size != 0:
        raise ValueError(f"sequence length ({seq_len}) not divisible by cp_size ({cp_size})")
    width = seq_len // cp_size
    return cp_rank * width, (cp_rank + 1) * width


def _check(x: Tensor, seq_dim: int) -> None:
    if x.dim() < 2:
        raise ValueError(f"CP tensor must have dim >= 2, got dim={x.dim()}")
    if not 0 <= seq_dim < x.dim():
        raise ValueError(f"seq_dim ({seq_dim}) out of range for {x.dim()}-dim tensor")


def _check_divisible(seq_len: int, cp_size: int) -> None:
    if cp_size < 1:
        raise ValueError(f"cp_size must be >= 1, got {cp_size}")
    if seq_len % cp_size != 0:
        raise ValueError(f"sequence length ({seq_len}) not divisible by cp_size ({cp_size})")


class _ScatterToContextParallelRegion(torch.autograd.Function):
    """Forward narrows to the local shard; backward zero-pads (no collective:
    each rank owns only the gradient of its own shard of the embedding)."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, group: Any, backend: CommBackend, cp_rank: int, cp_size: int, seq_dim: int):
        if cp_size == 1:
            ctx.meta = (cp_rank, cp_size, seq_dim, 0)
            return x
        _check(x, seq_dim)
        _check_divisible(x.size(seq_dim), cp_size)
        ctx.meta = (cp_rank, cp_size, seq_dim, x.size(seq_dim))
        width = x.size(seq_dim) // cp_size
        return x.narrow(seq_dim, cp_rank * width, width).contiguous()

    @staticmethod
    def backward(ctx: Any, grad: Tensor):
        cp_rank, cp_size, seq_dim, full = ctx.meta
        if cp_size == 1:
            return grad, None, None, None, None, None
        shape = list(grad.shape)
        shape[seq_dim] = full
        padded = grad.new_zeros(shape)
        width = full // cp_size
        padded.narrow(seq_dim, cp_rank * width, width).copy_(grad)
        return padded, None, None, None, None, None


class _GatherFromContextParallelRegion(torch.autograd.Function):
    """Forward: one single-buffer all-gather along the sequence.  Backward:
    reduce-scatter (partial contributions) or split (identical consumers)."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, group: Any, backend: CommBackend, cp_rank: int, cp_size: int, seq_dim: int,
                grad_op: str):
        ctx.meta = (group, backend, cp_rank, cp_size, seq_dim, grad_op)
        if cp_size == 1:
            return x
        _check(x, seq_dim)
        seq_first = x.movedim(seq_dim, 0).contiguous()
        out = seq_first.new_empty((seq_first.shape[0] * cp_size, *seq_first.shape[1:]))
        backend.all_gather_into_tensor(out, seq_first, group=group)
        return out.movedim(0, seq_dim)

    @staticmethod
    def backward(ctx: Any, grad: Tensor):
        group, backend, cp_rank, cp_size, seq_dim, grad_op = ctx.meta
        if cp_size == 1:
            return grad, None, None, None, None, None, None
        _check_divisible(grad.size(seq_dim), cp_size)
        if grad_op == "split":
            width = grad.size(seq_dim) // cp_size
            return grad.narrow(seq_dim, cp_rank * width, width).contiguous(), None, None, None, None, None, None
        pieces = [c.contiguous() for c in grad.chunk(cp_size, dim=seq_dim)]
        out = torch.empty_like(pieces[0])
        backend.reduce_scatter(out, pieces, group=group, op="sum")
        return out, None, None, None, None, None, None


def scatter_to_context_parallel_region(x: Tensor, group: Any, backend: CommBackend, cp_rank: int, cp_size: int, *,
                                       seq_dim: int = 1) -> Tensor:
    return _ScatterToContextParallelRegion.apply(x, group, backend, cp_rank, cp_size, seq_dim)


def gather_from_context_parallel_region(x: Tensor, group: Any, backend: CommBackend, cp_rank: int, cp_size: int, *,
                                        seq_dim: int = 1, grad_op: str = "reduce_scatter") -> Tensor:
    if grad_op not in ("reduce_scatter", "split"):
        raise ValueError(f"grad_op must be 'reduce_scatter' or 'split', got {grad_op!r}")
    return _GatherFromContextParallelRegion.apply(x, group, backend, cp_rank, cp_size, seq_dim, grad_op)


def causal_attn_scores_cp(q: Tensor, k_full: Tensor, scale: float, query_start: int) -> Tensor:
    """Scores of a local query shard ``[B,h,S_loc,d]`` (first row at global
    position ``query_start``) against the full keys, future keys masked with
    the dtype's minimum."""
    scores = torch.matmul(q, k_full.transpose(-2, -1)) * scale
    q_pos = torch.arange(query_start, query_start + q.size(2), device=scores.device).unsqueeze(1)
    k_pos = torch.arange(k_full.size(2), device=scores.device).unsqueeze(0)
    return scores.masked_fill((k_pos > q_pos)[None, None], torch.finfo(scores.dtype).min)
