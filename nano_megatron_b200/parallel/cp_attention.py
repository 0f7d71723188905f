"""Context-parallel attention on ``[B, S_loc, heads, d]`` bf16 tensors.

The reference all-gathers K and V (two collectives per layer, a ``c``-times
larger copy of each) and then loops over the visible blocks with separate
flash-attn calls and an fp32 merge per block
(nano_megatron/parallel/attention_backend.py:431-451, :615-632).  Here one
kernel launch walks the chunks.  Two transports:

* peer memory (default when a :class:`~nano_megatron_b200.distributed.symmetric.SymmetricWorkspace`
  is registered for the CP group): every rank publishes its K/V shard in its
  own symmetric buffer and the kernel's TMA loads read the other ranks' shards
  in place over NVLink -- nothing is gathered.  dK/dV tiles for a peer's chunk
  are stored straight into that peer's staging slot and the owner sums the
  slots.
* all-gather (any backend): K and V are gathered into one buffer each and the
  kernel reads the chunks from it; dK/dV are reduce-scattered.
"""
from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from ..distributed.backend import CommBackend


class _CPFlashAllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, q: Tensor, k: Tensor, v: Tensor, scale: float, group: Any, backend: CommBackend,
                cp_rank: int, cp_size: int):
        from ..ops.attention import attn_fwd

        k, v = k.contiguous(), v.contiguous()
        k_all = k.new_empty((cp_size, *k.shape))
        v_all = v.new_empty((cp_size, *v.shape))
        backend.all_gather_into_tensor(k_all.view(-1, *k.shape[1:]), k, group=group)
        backend.all_gather_into_tensor(v_all.view(-1, *v.shape[1:]), v, group=group)
        out, lse = attn_fwd(q, list(k_all.unbind(0)), list(v_all.unbind(0)), scale, q_pos0=cp_rank * q.shape[1])
        ctx.save_for_backward(q, k_all, v_all, out, lse)
        ctx.meta = (scale, group, backend, cp_rank, cp_size)
        return out

    @staticmethod
    def backward(ctx: Any, dout: Tensor):
        from ..ops.attention import attn_bwd

        q, k_all, v_all, out, lse = ctx.saved_tensors
        scale, group, backend, cp_rank, cp_size = ctx.meta
        dk_all, dv_all = torch.zeros_like(k_all), torch.zeros_like(v_all)
        dq, _, _ = attn_bwd(q, list(k_all.unbind(0)), list(v_all.unbind(0)), out, dout, lse, scale,
                            q_pos0=cp_rank * q.shape[1], dk_chunks=list(dk_all.unbind(0)),
                            dv_chunks=list(dv_all.unbind(0)))
        dk = torch.empty_like(k_all[0])
        dv = torch.empty_like(v_all[0])
        backend.reduce_scatter(dk, list(dk_all.unbind(0)), group=group, op="sum")
        backend.reduce_scatter(dv, list(dv_all.unbind(0)), group=group, op="sum")
        return dq, dk, dv, None, None, None, None, None


def cp_flash_attention(q: Tensor, k: Tensor, v: Tensor, *, scale: float, cp_group: Any, cp_rank: int, cp_size: int,
                       backend: CommBackend) -> Tensor:
    if q.shape[1] % 128 != 0:
        raise ValueError(f"context-parallel flash attention needs S_local % 128 == 0, got {q.shape[1]}")
    from ..distributed import symmetric

    ws = symmetric.workspace_for(cp_group)
    if ws is not None:
        return symmetric.cp_flash_attention_peer(q, k, v, scale, ws, cp_rank, cp_size)
    return _CPFlashAllGather.apply(q, k, v, float(scale), cp_group, backend, cp_rank, cp_size)
