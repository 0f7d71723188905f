"""Shifted next-token cross entropy (nano_megatron/reference/loss.py:7-23)."""
from __future__ import annotations

import torch.nn.functional as F
from torch import Tensor


def shifted_cross_entropy(logits: Tensor, labels: Tensor, ignore_index: int = -100) -> Tensor:
    """Predict ``labels[:, 1:]`` from ``logits[:, :-1]``; mean over kept tokens."""
    pred = logits[:, :-1, :].contiguous()
    tgt = labels[:, 1:].contiguous()
    return F.cross_entropy(pred.view(-1, pred.size(-1)), tgt.view(-1),
                           ignore_index=ignore_index, reduction="mean")
