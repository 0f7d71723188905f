"""Vocabulary-parallel embedding and cross entropy.

API as in the reference (nano_megatron/parallel/vocab_parallel.py:19-267).  On
bf16 CUDA tensors the embedding is one gather kernel that already produces zero
rows for ids outside the shard, and the loss is the fused CE of
``csrc/cross_entropy.cu``: one pass for (max, sum-exp, target logit), ONE
all-gather of three floats per token in place of the reference's three
all-reduces (:118-140), fp32 statistics, and a backward that recomputes the
softmax from the logits instead of saving a ``[N, V/t]`` tensor.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
from torch import Tensor, nn

from ..distributed.backend import CommBackend
from ..ops import functional as OF
from .mappings import _ReduceFromTPRegion


def vocab_range_from_global(rank: int, tp_size: int, vocab_size: int) -> tuple[int, int]:
    if tp_size < 1:
        raise ValueError(f"tp_size must be >= 1, got {tp_size}")
    if not 0 <= rank < tp_size:
        raise ValueError(f"rank ({rank}) out of range for tp_size ({tp_size})")
    if vocab_size < 1:
        raise ValueError(f"vocab_size must be >= 1, got {vocab_size}")
    if vocab_size % tp_size != 0:
        raise ValueError(
            f"vocab_size ({vocab_size}) not divisible by tp_size ({tp_size}); v1 requires an even vocab split")
    per = vocab_size // tp_size
    return rank * per, (rank + 1) * per


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, *, tp_rank: int, tp_size: int, group: Any,
                 backend: CommBackend, weight: Optional[Tensor] = None) -> None:
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.group, self.backend = group, backend
        self.vocab_start_index, self.vocab_end_index = vocab_range_from_global(tp_rank, tp_size, num_embeddings)
        if weight is not None:
            if tuple(weight.shape) != (num_embeddings, embedding_dim):
                raise ValueError(f"weight shape {tuple(weight.shape)} != ({num_embeddings}, {embedding_dim})")
            local = weight.data[self.vocab_start_index:self.vocab_end_index, :].clone()
        else:
            local = torch.empty(self.vocab_end_index - self.vocab_start_index, embedding_dim)
            nn.init.normal_(local)
        self.weight = nn.Parameter(local)

    def forward(self, input_ids: Tensor, *, positions: Optional[Tensor] = None,
                pos_weight: Optional[Tensor] = None) -> Tensor:
        """Lookup + sum over the TP group.  ``pos_weight`` (replicated position
        table) is folded into the same kernel when there is nothing to reduce."""
        fuse_pos = pos_weight is not None and self.tp_size == 1
        out = OF.embedding(input_ids, positions if fuse_pos else None, self.weight,
                           pos_weight if fuse_pos else None, self.vocab_start_index)
        if self.tp_size > 1:
            out = _ReduceFromTPRegion.apply(out, self.group, self.backend, None)
        if pos_weight is not None and not fuse_pos:
            out = out + torch.nn.functional.embedding(positions, pos_weight)
        return out


class _VocabParallelCrossEntropy(torch.autograd.Function):
    """Per-token CE over vocab-sharded logits, PyTorch path (CPU / fp32)."""

    @staticmethod
    def forward(ctx: Any, logits: Tensor, target: Tensor, vocab_start: int, vocab_end: int, ignore_index: int,
                group: Any, backend: CommBackend) -> Tensor:
        row_max = logits.max(dim=-1).values
        backend.all_reduce(row_max, group=group, op="max")
        shifted = logits - row_max.unsqueeze(-1)
        foreign = (target < vocab_start) | (target >= vocab_end)
        ignored = target == ignore_index
        local_idx = (target - vocab_start).masked_fill(foreign, 0)
        picked = shifted.gather(-1, local_idx.unsqueeze(-1)).squeeze(-1)
        picked = picked.masked_fill(foreign | ignored, 0.0)
        backend.all_reduce(picked, group=group, op="sum")
        exps = shifted.exp()
        denom = exps.sum(dim=-1)
        backend.all_reduce(denom, group=group, op="sum")
        loss = (torch.log(denom) - picked).masked_fill(ignored, 0.0)
        ctx.save_for_backward(exps / denom.unsqueeze(-1), target)
        ctx.meta = (vocab_start, vocab_end, ignore_index)
        return loss

    @staticmethod
    def backward(ctx: Any, grad_out: Tensor):
        probs, target = ctx.saved_tensors
        vocab_start, vocab_end, ignore_index = ctx.meta
        ignored = target == ignore_index
        mine = (target >= vocab_start) & (target < vocab_end) & ~ignored
        grad = probs * grad_out.unsqueeze(-1)
        local_idx = (target - vocab_start).masked_fill(~mine, 0)
        rows = torch.arange(target.size(0), device=target.device)
        grad[rows, local_idx] -= torch.where(mine, grad_out, torch.zeros_like(grad_out))
        grad = grad.masked_fill(ignored.unsqueeze(-1), 0.0)
        return grad, None, None, None, None, None, None


def vocab_parallel_cross_entropy_from_shifted(shift_logits: Tensor, shift_labels: Tensor, *, vocab_start_index: int,
                                              vocab_end_index: int, group: Any, backend: CommBackend,
                                              ignore_index: int = -100, reduction: str = "mean",
                                              tp_size: Optional[int] = None) -> Tensor:
    """CE over already-paired ``[B, T, V/t]`` logits and ``[B, T]`` labels."""
    if reduction not in ("mean", "sum"):
        raise ValueError(f"reduction must be 'mean' or 'sum', got {reduction!r}")
    if shift_logits.dim() != 3:
        raise ValueError(f"expected shift_logits [B, T, local_V], got shape {tuple(shift_logits.shape)}")
    if shift_labels.shape != shift_logits.shape[:2]:
        raise ValueError(f"shift_labels shape {tuple(shift_labels.shape)} incompatible with shift_logits "
                         f"{tuple(shift_logits.shape)}")
    vloc = shift_logits.size(-1)
    logits2d = shift_logits.reshape(-1, vloc)
    labels1d = shift_labels.reshape(-1)
    if OF.use_native(logits2d):
        if tp_size is None:
            tp_size = 1 if vocab_end_index - vocab_start_index == vloc and group is None else _group_size(group)
        total, count = OF.cross_entropy_sum(logits2d, labels1d, vocab_start=vocab_start_index,
                                            ignore_index=ignore_index, group=group, backend=backend, tp_size=tp_size)
        if reduction == "sum":
            return total
        return total / torch.clamp(count, min=1.0)
    per_token = _VocabParallelCrossEntropy.apply(logits2d, labels1d, vocab_start_index, vocab_end_index,
                                                 ignore_index, group, backend)
    valid = labels1d != ignore_index
    if not valid.any():
        return per_token.sum() * 0.0
    return per_token[valid].sum() if reduction == "sum" else per_token[valid].mean()


def _group_size(group: Any) -> int:
    import torch.distributed as dist
    if group is None and not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def vocab_parallel_cross_entropy(vocab_parallel_logits: Tensor, target: Tensor, *, vocab_start_index: int,
                                 vocab_end_index: int, group: Any, backend: CommBackend,
                                 ignore_index: int = -100, tp_size: Optional[int] = None) -> Tensor:
    """Shifted CE (predict ``target[:, 1:]`` from ``logits[:, :-1]``), mean over kept tokens."""
    if vocab_parallel_logits.dim() != 3:
        raise ValueError(f"expected logits [B, S, local_V], got shape {tuple(vocab_parallel_logits.shape)}")
    if target.shape != vocab_parallel_logits.shape[:2]:
        raise ValueError(f"target shape {tuple(target.shape)} incompatible with logits "
                         f"{tuple(vocab_parallel_logits.shape)}")
    if OF.use_native(vocab_parallel_logits):
        # No shifted copy of the logits: the last position of every sequence is
        # given the ignore label instead, which removes it from loss and count.
        labels = torch.full_like(target, ignore_index)
        labels[:, :-1] = target[:, 1:]
        return vocab_parallel_cross_entropy_from_shifted(
            vocab_parallel_logits, labels, vocab_start_index=vocab_start_index, vocab_end_index=vocab_end_index,
            group=group, backend=backend, ignore_index=ignore_index, reduction="mean", tp_size=tp_size)
    return vocab_parallel_cross_entropy_from_shifted(
        vocab_parallel_logits[:, :-1, :].contiguous(), target[:, 1:].contiguous(),
        vocab_start_index=vocab_start_index, vocab_end_index=vocab_end_index, group=group, backend=backend,
        ignore_index=ignore_index, reduction="mean", tp_size=tp_size)
