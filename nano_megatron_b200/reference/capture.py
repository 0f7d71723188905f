"""Detached CPU snapshots of parameters, gradients, optimizer state and
activation trees (nano_megatron/reference/capture.py:12-54)."""
from __future__ import annotations

from typing import Any, Literal

from torch import Tensor
from torch.nn import Module

CaptureLevel = Literal["minimal", "grads", "full"]


def _host_copy(t: Tensor) -> Tensor:
    return t.detach().to(device="cpu", dtype=t.dtype).clone()


def snapshot_tree(obj: Any) -> Any:
    if isinstance(obj, Tensor):
        return _host_copy(obj)
    if isinstance(obj, dict):
        return {k: snapshot_tree(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(snapshot_tree(v) for v in obj)
    return obj


def snapshot_params(model: Module) -> dict[str, Tensor]:
    return {n: _host_copy(p) for n, p in model.named_parameters()}


def snapshot_grads(model: Module) -> dict[str, Tensor]:
    grads: dict[str, Tensor] = {}
    for n, p in model.named_parameters():
        if p.grad is None:
            raise RuntimeError(f"missing grad for parameter {n!r}")
        grads[n] = _host_copy(p.grad)
    return grads


def snapshot_optimizer(opt: Any) -> dict[str, dict[str, Any]]:
    return {
        n: {"exp_avg": _host_copy(e["exp_avg"]), "exp_avg_sq": _host_copy(e["exp_avg_sq"]), "step": int(e["step"])}
        for n, e in opt.state_dict().items()
    }
