"""AdamW with state keyed by parameter name.

Semantics follow ``torch.optim.AdamW`` (decoupled weight decay, bias
correction) and the state layout ``{name: {"exp_avg", "exp_avg_sq", "step"}}``
follows nano_megatron/reference/optimizer.py:13-131.  On CPU the update is the
reference's per-parameter sequence of PyTorch ops (bit-identical to it); on a
CUDA device every parameter of the model is updated by ONE launch of the fused
multi-tensor kernel (``csrc/adamw.cu``) that reads grad / param / moments once
and writes param / moments once.
"""
from __future__ import annotations

from collections.abc import Iterable
from typing import Any

import torch
from torch import Tensor
from torch.nn import Parameter


class AdamW:
    def __init__(
        self,
        named_params: Iterable[tuple[str, Parameter]],
        lr: float,
        betas: tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 0.0,
    ) -> None:
        self.state: dict[str, dict[str, Any]] = {}
        self.lr = float(lr)
        self.betas = (float(betas[0]), float(betas[1]))
        self.eps = float(eps)
        self.weight_decay = float(weight_decay)
        self._params: list[tuple[str, Parameter]] = []
        names: set[str] = set()
        for name, param in named_params:
            if name in names:
                raise ValueError(f"duplicate parameter name: {name!r}")
            if not isinstance(param, Parameter):
                raise TypeError(f"expected Parameter for {name!r}, got {type(param)}")
            names.add(name)
            self._params.append((name, param))
        self._fused = None  # most recently used device-side plan
        self._plans: dict = {}

    # ---------------------------------------------------------------- step --
    def _ensure_state(self, name: str, param: Parameter) -> dict[str, Any]:
        st = self.state.get(name)
        if st is None:
            st = {
                "step": 0,
                "exp_avg": torch.zeros_like(param, dtype=torch.float32),
                "exp_avg_sq": torch.zeros_like(param, dtype=torch.float32),
            }
            self.state[name] = st
        return st

    def step(self, *, only: "set[int] | None" = None, exclude: "set[int] | None" = None) -> None:
        """Update every parameter that has a gradient.  ``only`` / ``exclude``
        (sets of ``id(param)``) restrict the update to a subset, so that a caller
        can update most parameters while the gradients of the rest are still
        being reduced, and those afterwards."""
        live = [(n, p) for n, p in self._params if p.grad is not None
                and (only is None or id(p) in only) and (exclude is None or id(p) not in exclude)]
        if not live:
            return
        for n, p in live:
            if p.grad.is_sparse:
                raise RuntimeError(f"AdamW does not support sparse gradients ({n!r})")
        if all(p.is_cuda for _, p in live):
            self._step_fused(live)
        else:
            for n, p in live:
                self._step_one(n, p)

    def _step_one(self, name: str, param: Parameter) -> None:
        b1, b2 = self.betas
        st = self._ensure_state(name, param)
        st["step"] = int(st["step"]) + 1
        t = st["step"]
        m: Tensor = st["exp_avg"]
        v: Tensor = st["exp_avg_sq"]
        data = param.data
        w = data if data.dtype == torch.float32 else data.float()
        g = param.grad.detach()
        g = g if g.dtype == torch.float32 else g.float()
        if self.weight_decay != 0.0:
            w = w.mul(1.0 - self.lr * self.weight_decay)
        m.mul_(b1).add_(g, alpha=1.0 - b1)
        v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
        corr1 = 1.0 - b1 ** t
        corr2 = 1.0 - b2 ** t
        denom = (v.sqrt() / (corr2 ** 0.5)).add_(self.eps)
        w = w.addcdiv(m, denom, value=-(self.lr / corr1))
        data.copy_(w if data.dtype == torch.float32 else w.to(dtype=data.dtype))

    def _step_fused(self, live: list[tuple[str, Parameter]]) -> None:
        from ..ops.adamw import FusedAdamWPlan

        key = tuple((n, p.data_ptr(), p.grad.data_ptr()) for n, p in live)
        plan = self._plans.get(key)
        if plan is None:
            # a plan per distinct parameter subset (the whole model, one gradient bucket, ...)
            states = [self._ensure_state(n, p) for n, p in live]
            plan = FusedAdamWPlan(key, [p for _, p in live], states)
            plan.names = [n for n, _ in live]
            if len(self._plans) >= 512:          # one per gradient bucket at most, in practice
                self._plans.clear()
            self._plans[key] = plan
        self._fused = plan
        plan.step(self.lr, self.betas, self.eps, self.weight_decay)
        for n, _ in live:
            # `step` is mirrored on the host so state_dict() needs no sync.
            self.state[n]["step"] = int(self.state[n]["step"]) + 1

    def zero_grad(self, set_to_none: bool = True) -> None:
        for _, p in self._params:
            if p.grad is None:
                continue
            if set_to_none:
                p.grad = None
            else:
                p.grad.detach_()
                p.grad.zero_()

    # ---------------------------------------------------------- state dict --
    def _sync_step_from_device(self) -> None:
        """A replayed CUDA graph advances the device step counter only."""
        for plan in self._plans.values():
            done = int(plan.step_count.item())
            for n in plan.names:
                self.state[n]["step"] = done

    def state_dict(self) -> dict[str, dict[str, Any]]:
        self._sync_step_from_device()
        return {
            n: {"exp_avg": s["exp_avg"].clone(), "exp_avg_sq": s["exp_avg_sq"].clone(), "step": int(s["step"])}
            for n, s in self.state.items()
        }

    def load_state_dict(self, state: dict[str, dict[str, Any]]) -> None:
        """Load moments and step counts.  Existing state tensors of matching
        shape are overwritten *in place* (and the fused plan's device-side step
        counter with them), so device addresses baked into a captured CUDA
        graph of the step stay valid and the replayed graph sees the loaded
        state."""
        by_name = dict(self._params)
        fresh: dict[str, dict[str, Any]] = {}
        in_place = True
        for n, entry in state.items():
            dev = by_name[n].device if n in by_name else entry["exp_avg"].device
            old = self.state.get(n)
            if (old is not None and old["exp_avg"].shape == entry["exp_avg"].shape
                    and old["exp_avg"].device == torch.device(dev)):
                old["exp_avg"].copy_(entry["exp_avg"].detach())
                old["exp_avg_sq"].copy_(entry["exp_avg_sq"].detach())
                old["step"] = int(entry["step"])
                fresh[n] = old
                continue
            in_place = False
            fresh[n] = {
                "exp_avg": entry["exp_avg"].detach().to(device=dev, dtype=torch.float32).clone(),
                "exp_avg_sq": entry["exp_avg_sq"].detach().to(device=dev, dtype=torch.float32).clone(),
                "step": int(entry["step"]),
            }
        if set(fresh) != set(self.state):
            in_place = False
        self.state = fresh
        if self._plans and in_place:
            ok = True
            for plan in self._plans.values():
                steps = {int(self.state[n]["step"]) for n in plan.names}
                if len(steps) == 1:
                    plan.step_count.fill_(steps.pop())
                else:
                    ok = False
            if ok:
                return
        self._fused = None
        self._plans.clear()

    def sync_hyper(self) -> None:
        """Push ``lr`` / betas / eps / weight decay to the fused plan's device
        copy if they changed on the host (a plain device copy; call it outside a
        captured graph, before replaying it)."""
        for plan in self._plans.values():
            plan.set_hyper(self.lr, self.betas, self.eps, self.weight_decay)
