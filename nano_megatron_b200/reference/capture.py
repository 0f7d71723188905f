"""Host-side snapshots (detached, cloned, same dtype) of parameters, gradients,
optimizer moments and nested activation containers; the entry points and the
"missing grad" error follow nano_megatron/reference/capture.py:12-54.
"""
from __future__ import annotations

from typing import Any, Callable, Literal

from torch import Tensor
from torch.nn import Module

CaptureLevel = Literal["minimal", "grads", "full"]


def _host_copy(t: Tensor) -> Tensor:
    return t.detach().to(device="cpu", dtype=t.dtype).clone()


def snapshot_tree(obj: Any) -> Any:
    """Tensors anywhere inside dicts / lists / tuples are replaced by host
    copies; the containers keep their types, other leaves pass through."""
    if isinstance(obj, Tensor):
        return _host_copy(obj)
    if isinstance(obj, dict):
        return {key: snapshot_tree(value) for key, value in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(snapshot_tree(item) for item in obj)
    return obj


def _per_parameter(model: Module, pick: Callable[[str, Tensor], Tensor]) -> dict[str, Tensor]:
    return {name: _host_copy(pick(name, param)) for name, param in model.named_parameters()}


def snapshot_params(model: Module) -> dict[str, Tensor]:
    return _per_parameter(model, lambda _name, param: param)


def snapshot_grads(model: Module) -> dict[str, Tensor]:
    def grad_of(name: str, param: Tensor) -> Tensor:
        if param.grad is None:
            raise RuntimeError(f"missing grad for parameter {name!r}")
        return param.grad

    return _per_parameter(model, grad_of)


def snapshot_optimizer(opt: Any) -> dict[str, dict[str, Any]]:
    """``{parameter name: {"exp_avg", "exp_avg_sq", "step"}}`` from ``opt.state_dict()``."""
    out: dict[str, dict[str, Any]] = {}
    for name, entry in opt.state_dict().items():
        out[name] = {"exp_avg": _host_copy(entry["exp_avg"]), "exp_avg_sq": _host_copy(entry["exp_avg_sq"]),
                     "step": int(entry["step"])}
    return out
