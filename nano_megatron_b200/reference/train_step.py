"""The oracle's optimisation step and loop on one device, with snapshots for
parity checks.  Public names, signatures, ``StepResult`` fields and error
messages follow nano_megatron/reference/train_step.py:25-120 (they are the
contract the parity tests use); the body is organised around a table of what
each capture level records.
"""
from __future__ import annotations

import random
from collections.abc import Sequence
from dataclasses import dataclass
from typing import Any, Optional

import torch
from torch import Tensor
from torch.nn import Module

from . import capture as _cap
from .capture import CaptureLevel
from .loss import shifted_cross_entropy
from .optimizer import AdamW

# capture level -> (record gradients, record activations + optimizer state)
_RECORDS: dict[str, tuple[bool, bool]] = {"minimal": (False, False), "grads": (True, False), "full": (True, True)}


@dataclass
class StepResult:
    """What one step leaves behind, all on the host.  ``params`` are the values
    AFTER the update, ``grads`` the gradients the update consumed."""

    step: int
    loss: Tensor
    logits: Tensor
    params: dict[str, Tensor]
    grads: Optional[dict[str, Tensor]] = None
    activations: Optional[dict[str, Any]] = None
    optimizer_state: Optional[dict[str, dict[str, Any]]] = None


def seed_all(seed: int) -> None:
    """Seed Python's and PyTorch's generators (every CUDA device included)."""
    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def reference_train_step(model: Module, optimizer: AdamW, input_ids: Tensor, labels: Optional[Tensor] = None,
                         capture_level: CaptureLevel = "full", step: int = 0) -> StepResult:
    if capture_level not in _RECORDS:
        raise ValueError(f"unknown capture_level: {capture_level!r}")
    with_grads, with_everything = _RECORDS[capture_level]

    optimizer.zero_grad(set_to_none=True)
    taps = None
    if with_everything:
        logits, taps = model.forward_with_activations(input_ids)
    else:
        logits = model.forward(input_ids)
    loss = shifted_cross_entropy(logits, labels if labels is not None else input_ids)
    loss.backward()

    extras: dict[str, Any] = {}
    if with_grads:
        extras["grads"] = _cap.snapshot_grads(model)       # before the update consumes them
    optimizer.step()
    if with_everything:
        extras["activations"] = _cap.snapshot_tree(taps)
        extras["optimizer_state"] = _cap.snapshot_optimizer(optimizer)
    return StepResult(step=step, loss=_cap.snapshot_tree(loss), logits=_cap.snapshot_tree(logits),
                      params=_cap.snapshot_params(model), **extras)


def reference_train_loop(model: Module, optimizer: AdamW, batches: Sequence[Tensor], steps: int,
                         capture_every: int = 1, capture_level: CaptureLevel = "full") -> list[StepResult]:
    """``steps`` updates over ``batches`` (cycled).  Every ``capture_every``-th
    step is run at ``capture_level`` and returned; the others run at "minimal"
    and are dropped."""
    if steps < 0:
        raise ValueError(f"steps must be non-negative, got {steps}")
    if capture_every < 1:
        raise ValueError(f"capture_every must be >= 1, got {capture_every}")
    if steps > 0 and len(batches) == 0:
        raise ValueError("batches is empty but steps > 0")
    history: list[StepResult] = []
    for index in range(steps):
        recorded = index % capture_every == 0
        outcome = reference_train_step(model, optimizer, batches[index % len(batches)],
                                       capture_level=capture_level if recorded else "minimal", step=index)
        if recorded:
            history.append(outcome)
    return history
