"""Device-side plan for the fused multi-tensor AdamW (``csrc/adamw.cu``)."""
from __future__ import annotations

import ctypes
import struct
from typing import Any

import torch

from . import native


class FusedAdamWPlan:
    """Table of (param, grad, moments) pointers uploaded once; one launch per step.

    ``key`` identifies the set of tensors the table was built for so the owner
    can rebuild it if a gradient buffer moves.
    """

    def __init__(self, key: Any, params: list[torch.nn.Parameter], states: list[dict]) -> None:
        self.key = key
        lib = native.lib()
        lib.nmb_adamw_blocks_for.restype = ctypes.c_longlong
        entry = lib.nmb_adamw_table_entry_size()
        assert entry == 56, f"unexpected AdamTensor size {entry}"
        device = params[0].device
        raw = bytearray()
        first = 0
        for p, st in zip(params, states):
            g = p.grad
            assert g is not None and g.is_contiguous() and p.is_contiguous()
            assert p.dtype in (torch.bfloat16, torch.float32) and g.dtype in (torch.bfloat16, torch.float32)
            raw += struct.pack("<QQQQqqii", p.data_ptr(), g.data_ptr(), st["exp_avg"].data_ptr(),
                               st["exp_avg_sq"].data_ptr(), p.numel(), first,
                               int(p.dtype == torch.bfloat16), int(g.dtype == torch.bfloat16))
            first += int(lib.nmb_adamw_blocks_for(ctypes.c_longlong(p.numel())))
        self.total_blocks = first
        self.n = len(params)
        self.table = torch.frombuffer(raw, dtype=torch.uint8).clone().to(device)
        steps = {int(st["step"]) for st in states}
        if len(steps) != 1:
            raise RuntimeError("fused AdamW needs all parameters at the same step count")
        self.step_count = torch.tensor([steps.pop()], dtype=torch.int32, device=device)
        self.hyper = torch.zeros(5, dtype=torch.float32, device=device)
        self._hyper_host: tuple | None = None
        self._keep = (params, states)

    def set_hyper(self, lr: float, betas: tuple[float, float], eps: float, weight_decay: float) -> None:
        """Refresh the device copy of the hyper-parameters if they changed."""
        hv = (lr, betas[0], betas[1], eps, weight_decay)
        if hv != self._hyper_host:
            self.hyper.copy_(torch.tensor(hv, dtype=torch.float32))
            self._hyper_host = hv

    def step(self, lr: float, betas: tuple[float, float], eps: float, weight_decay: float) -> None:
        self.set_hyper(lr, betas, eps, weight_decay)
        rc = native.lib().nmb_adamw_step(native.ptr(self.table), ctypes.c_int(self.n),
                                         ctypes.c_longlong(self.total_blocks), native.ptr(self.hyper),
                                         native.ptr(self.step_count), native.stream_ptr(self.table.device))
        native.check_rc(rc, "nmb_adamw_step")
