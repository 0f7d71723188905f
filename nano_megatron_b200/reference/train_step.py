"""One-device training step / loop with optional capture
(nano_megatron/reference/train_step.py:25-120)."""
from __future__ import annotations

import random
from collections.abc import Sequence
from dataclasses import dataclass
from typing import Any, Optional

import torch
from torch import Tensor
from torch.nn import Module

from .capture import CaptureLevel, snapshot_grads, snapshot_optimizer, snapshot_params, snapshot_tree
from .loss import shifted_cross_entropy
from .optimizer import AdamW


@dataclass
class StepResult:
    step: int
    loss: Tensor
    logits: Tensor
    params: dict[str, Tensor]
    grads: Optional[dict[str, Tensor]] = None
    activations: Optional[dict[str, Any]] = None
    optimizer_state: Optional[dict[str, dict[str, Any]]] = None


def seed_all(seed: int) -> None:
    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def reference_train_step(
    model: Module,
    optimizer: AdamW,
    input_ids: Tensor,
    labels: Optional[Tensor] = None,
    capture_level: CaptureLevel = "full",
    step: int = 0,
) -> StepResult:
    if capture_level not in ("minimal", "grads", "full"):
        raise ValueError(f"unknown capture_level: {capture_level!r}")
    targets = input_ids if labels is None else labels
    optimizer.zero_grad(set_to_none=True)
    raw_acts = None
    if capture_level == "full":
        logits, raw_acts = model.forward_with_activations(input_ids)
    else:
        logits = model.forward(input_ids)
    loss = shifted_cross_entropy(logits, targets)
    loss.backward()
    grads = snapshot_grads(model) if capture_level in ("grads", "full") else None
    optimizer.step()
    result = StepResult(
        step=step,
        loss=loss.detach().cpu().clone(),
        logits=logits.detach().cpu().clone(),
        params=snapshot_params(model),
        grads=grads,
    )
    if capture_level == "full":
        result.activations = snapshot_tree(raw_acts)
        result.optimizer_state = snapshot_optimizer(optimizer)
    return result


def reference_train_loop(
    model: Module,
    optimizer: AdamW,
    batches: Sequence[Tensor],
    steps: int,
    capture_every: int = 1,
    capture_level: CaptureLevel = "full",
) -> list[StepResult]:
    if steps < 0:
        raise ValueError(f"steps must be non-negative, got {steps}")
    if capture_every < 1:
        raise ValueError(f"capture_every must be >= 1, got {capture_every}")
    if len(batches) == 0 and steps > 0:
        raise ValueError("batches is empty but steps > 0")
    kept: list[StepResult] = []
    for i in range(steps):
        keep = i % capture_every == 0
        res = reference_train_step(
            model, optimizer, batches[i % len(batches)], labels=None,
            capture_level=capture_level if keep else "minimal", step=i,
        )
        if keep:
            kept.append(res)
    return kept
