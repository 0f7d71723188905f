"""Gradient buckets for data-parallel synchronisation.

API of the reference's ``GradBucket`` / ``build_buckets``
(nano_megatron/distributed/bucket.py:12-152): parameters in reverse
registration order, a new bucket on a dtype change or when the byte cap would
be exceeded, ``mark_ready`` / ``sync`` / ``reset``.

Unlike the reference, a bucket can own a *persistent* flat buffer
(:meth:`GradBucket.bind_persistent`): the parameters' ``.grad`` (and
``main_grad``) are views into it, so ``sync`` reduces the buffer in place and
the flatten / ``div_`` / unflatten passes over every gradient
(reference :85-100) disappear.  Without a persistent buffer ``sync`` behaves
as the reference does (gather into a temporary, all-reduce, divide, copy back).
"""
from __future__ import annotations

from typing import Any, Callable, Optional

import torch
import torch.nn as nn
from torch import Tensor

from .backend import CommBackend


class GradBucket:
    def __init__(self, params: list[nn.Parameter]) -> None:
        if not params:
            raise ValueError("GradBucket requires at least one parameter")
        self._params = list(params)
        self._slot = {id(p): i for i, p in enumerate(self._params)}
        self._ready: set[int] = set()
        self._coalesced = False
        self._flat: Optional[Tensor] = None
        self._persistent: Optional[Tensor] = None
        self._views: list[Tensor] = []
        #: optional device-side reducer ``fn(flat, divisor)``; when it returns
        #: True the bucket was reduced and scaled by it.
        self.fused_reduce: Optional[Callable[[Tensor, int], bool]] = None

    # ------------------------------------------------------------ properties --
    @property
    def params(self) -> list[nn.Parameter]:
        return list(self._params)

    @property
    def coalesced(self) -> bool:
        return self._coalesced

    @property
    def has_pending_ready(self) -> bool:
        return bool(self._ready)

    @property
    def persistent_buffer(self) -> Optional[Tensor]:
        return self._persistent

    def numel(self) -> int:
        return sum(p.numel() for p in self._params)

    # ------------------------------------------------------------ persistent --
    def bind_persistent(self, flat: Tensor) -> None:
        """Make ``flat`` (1-D, this bucket's dtype, ``numel()`` long, zeroed) the
        home of the gradients: ``p.grad`` and ``p.main_grad`` become views."""
        if flat.numel() != self.numel():
            raise ValueError(f"persistent buffer has {flat.numel()} elements, bucket needs {self.numel()}")
        self._persistent = flat
        self._views = []
        offset = 0
        for p in self._params:
            view = flat[offset:offset + p.numel()].view_as(p)
            offset += p.numel()
            if p.grad is not None:
                view.copy_(p.grad)
            p.grad = view
            p.main_grad = view
            self._views.append(view)

    def _rehome_strays(self) -> None:
        """A caller may have set ``p.grad = None`` (so autograd made a fresh
        tensor): fold such gradients back into the persistent views."""
        for p, view in zip(self._params, self._views):
            g = p.grad
            if g is None:
                p.grad = view
            elif g.data_ptr() != view.data_ptr():
                view.add_(g)
                p.grad = view

    # ------------------------------------------------------------------ sync --
    def mark_ready(self, param: nn.Parameter) -> bool:
        slot = self._slot.get(id(param))
        if slot is None:
            raise KeyError("parameter not in this bucket")
        if self._coalesced or slot in self._ready:
            return False
        self._ready.add(slot)
        return len(self._ready) == len(self._params)

    def sync(self, backend: CommBackend, group: Any, dp_size: int, *, group_size: Optional[int] = None) -> None:
        """Sum over ``group`` and divide by ``dp_size`` (the mean divisor).

        ``group_size`` is the size of the communicating group, used only to skip
        the collective when it is 1; it defaults to ``dp_size``.  Pure context
        parallelism (``dp_size == 1``, ``group_size == cp``) still all-reduces.
        """
        if self._coalesced:
            return
        if self._persistent is not None:
            self._rehome_strays()
        missing = [p for p in self._params if p.grad is None]
        if missing:
            raise RuntimeError(
                f"GradBucket.sync: {len(missing)} parameter(s) have grad=None (unused params not supported)")
        divisor = dp_size
        if group_size is None:
            group_size = divisor
        if divisor < 1 or group_size < 1:
            raise ValueError(f"mean_divisor and group_size must be >= 1, got mean_divisor={divisor}, "
                             f"group_size={group_size}")
        if group_size == 1:
            self._coalesced = True
            return
        if self._persistent is not None:
            flat = self._persistent
            if self.fused_reduce is None or not self.fused_reduce(flat, divisor):
                backend.all_reduce(flat, group=group, op="sum")
                if divisor != 1:
                    flat.div_(divisor)
        else:
            grads = [p.grad for p in self._params]
            flat = torch.cat([g.reshape(-1) for g in grads])
            backend.all_reduce(flat, group=group, op="sum")
            flat.div_(divisor)
            offset = 0
            for g in grads:
                g.copy_(flat[offset:offset + g.numel()].view_as(g))
                offset += g.numel()
        self._flat = flat
        self._coalesced = True

    def reset(self) -> None:
        self._ready.clear()
        self._coalesced = False
        self._flat = None


def build_buckets(module: nn.Module, bucket_cap_mb: float = 25.0) -> list[GradBucket]:
    if bucket_cap_mb <= 0:
        raise ValueError(f"bucket_cap_mb must be > 0, got {bucket_cap_mb}")
    cap = int(bucket_cap_mb * 1024 * 1024)
    params = [p for p in module.parameters() if p.requires_grad][::-1]
    if not params:
        return []
    devices = {p.device for p in params}
    if len(devices) > 1:
        raise RuntimeError(f"build_buckets: parameters span multiple devices: {devices}")
    buckets: list[GradBucket] = []
    group: list[nn.Parameter] = []
    size = 0
    for p in params:
        nbytes = p.numel() * p.element_size()
        if group and (p.dtype != group[-1].dtype or size + nbytes > cap):
            buckets.append(GradBucket(group))
            group, size = [], 0
        group.append(p)
        size += nbytes
    buckets.append(GradBucket(group))
    return buckets
