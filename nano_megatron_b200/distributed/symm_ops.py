"""Operators that read or write peers' symmetric buffers from inside compute kernels."""
from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from .symm_mem import CHANNEL_CP, SymmetricWorkspace


class _KVExchange:
    """Per-workspace pool of symmetric K/V slots (one pair per attention call of
    a forward pass, reused every step) and one dK/dV staging area."""

    def __init__(self, ws: SymmetricWorkspace) -> None:
        self.ws = ws
        self.slots: list[tuple[Tensor, Tensor]] = []
        self.cursor = 0
        self.staging: dict[tuple, tuple[Tensor, Tensor]] = {}

    def next_slot(self, like: Tensor) -> tuple[Tensor, Tensor]:
        if self.cursor == len(self.slots):
            k = self.ws.alloc_tensor(like.numel(), like.dtype).view(like.shape)
            v = self.ws.alloc_tensor(like.numel(), like.dtype).view(like.shape)
            self.slots.append((k, v))
        pair = self.slots[self.cursor]
        if pair[0].shape != like.shape:
            raise RuntimeError("context-parallel K/V shape changed between steps")
        self.cursor += 1
        return pair

    def stage(self, like: Tensor) -> tuple[Tensor, Tensor]:
        key = (tuple(like.shape), like.dtype)
        if key not in self.staging:
            n = self.ws.size * like.numel()
            dk = self.ws.alloc_tensor(n, like.dtype).view(self.ws.size, *like.shape)
            dv = self.ws.alloc_tensor(n, like.dtype).view(self.ws.size, *like.shape)
            self.staging[key] = (dk, dv)
        return self.staging[key]


def _exchange(ws: SymmetricWorkspace) -> _KVExchange:
    ex = getattr(ws, "_kv_exchange", None)
    if ex is None:
        ex = _KVExchange(ws)
        ws._kv_exchange = ex
    return ex


def begin_step(ws: SymmetricWorkspace) -> None:
    """Rewind the K/V slot cursor (called at the start of every forward pass)."""
    _exchange(ws).cursor = 0


class _CPFlashPeer(torch.autograd.Function):
    """Context-parallel attention whose kernel reads the peers' K/V in place.

    forward : publish K/V in this rank's symmetric slot, barrier, then ONE
              attention launch whose TMA loads fetch chunk c from rank c's slot.
    backward: ONE launch computes dQ and this rank's dK/dV contribution to every
              visible chunk, storing chunk c's tiles straight into slot
              [my_rank] of rank c's staging buffer; after a barrier each rank
              sums the slots of the ranks that can see it (rank >= own).
    """

    @staticmethod
    def forward(ctx: Any, q: Tensor, k: Tensor, v: Tensor, scale: float, ws: SymmetricWorkspace, cp_rank: int,
                cp_size: int):
        from ..ops.attention import attn_fwd

        ex = _exchange(ws)
        k_slot, v_slot = ex.next_slot(k)
        k_slot.copy_(k)
        v_slot.copy_(v)
        ws.barrier(CHANNEL_CP)                       # every rank's K/V is published
        ks = [ws.peer_view(k_slot, r) for r in range(cp_size)]
        vs = [ws.peer_view(v_slot, r) for r in range(cp_size)]
        out, lse = attn_fwd(q, ks, vs, scale, q_pos0=cp_rank * q.shape[1])
        ctx.save_for_backward(q, out, lse)
        ctx.kv = (k_slot, v_slot)
        ctx.meta = (scale, ws, cp_rank, cp_size)
        return out

    @staticmethod
    def backward(ctx: Any, dout: Tensor):
        from ..ops.attention import attn_bwd

        q, out, lse = ctx.saved_tensors
        k_slot, v_slot = ctx.kv
        scale, ws, cp_rank, cp_size = ctx.meta
        ex = _exchange(ws)
        dk_stage, dv_stage = ex.stage(k_slot)
        ks = [ws.peer_view(k_slot, r) for r in range(cp_size)]
        vs = [ws.peer_view(v_slot, r) for r in range(cp_size)]
        # chunk c's gradient tiles go to slot [cp_rank] of rank c's staging buffer
        dks = [ws.peer_view(dk_stage, r)[cp_rank] for r in range(cp_size)]
        dvs = [ws.peer_view(dv_stage, r)[cp_rank] for r in range(cp_size)]
        ws.barrier(CHANNEL_CP)                       # the staging area is free (previous layer consumed it)
        dq, _, _ = attn_bwd(q, ks, vs, out, dout, lse, scale, q_pos0=cp_rank * q.shape[1], dk_chunks=dks,
                            dv_chunks=dvs)
        ws.barrier(CHANNEL_CP)                       # all contributions have landed
        dk = dk_stage[cp_rank:].float().sum(0).to(k_slot.dtype)
        dv = dv_stage[cp_rank:].float().sum(0).to(v_slot.dtype)
        return dq, dk, dv, None, None, None, None


def cp_flash_attention_peer(q: Tensor, k: Tensor, v: Tensor, scale: float, ws: SymmetricWorkspace, cp_rank: int,
                            cp_size: int) -> Tensor:
    return _CPFlashPeer.apply(q, k.contiguous(), v.contiguous(), float(scale), ws, cp_rank, cp_size)
