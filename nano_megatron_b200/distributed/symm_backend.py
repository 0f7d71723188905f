"""``CommBackend`` on this package's peer-memory kernels.

The reference's distributed layer is one protocol (nano_megatron/distributed/backend.py:8-47)
with one implementation on ``torch.distributed``.  :class:`SymmetricBackend` is a second
implementation of the same eight methods: for every process group that has a symmetric-memory
workspace (``enable_symmetric_memory``) the collectives run as plain CUDA kernels over peer
memory (two-shot all-reduce, peer-store all-gather, device barrier), so they can be captured
in a CUDA graph and involve no library communicator; everything else (CPU tensors, groups
without a workspace, point-to-point, reduce ops other than ``sum``, tensors larger than the
staging limit) goes to the wrapped ``torch.distributed`` backend, method by method.

The fused paths of the framework (GEMM + collective in one kernel, bucket reductions in
persistent symmetric buffers) do not go through this class: they own their buffers.  This
class is for the generic calls of user code and of the framework's cold paths, which work on
ordinary tensors and therefore pay one copy into a symmetric staging buffer and one copy out.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist
from torch import Tensor

from . import symmetric
from .symm_mem import CHANNEL_AUX
from .torch_backend import TorchDistBackend

#: tensors above this size use the library collective (the staging buffers come out of the
#: workspace's arenas and are kept)
STAGING_LIMIT_BYTES = 64 << 20


class _Done:
    """Handle of a collective that is already ordered on the current stream."""

    def wait(self) -> bool:
        return True

    def is_completed(self) -> bool:
        return True


class SymmetricBackend(TorchDistBackend):
    def __init__(self) -> None:
        #: how many calls ran on peer-memory kernels / on the library, per method
        self.counts: dict[str, int] = {}

    # ------------------------------------------------------------- helpers --
    def _count(self, method: str, symmetric_path: bool) -> None:
        key = f"{method}:{'symmetric' if symmetric_path else 'library'}"
        self.counts[key] = self.counts.get(key, 0) + 1

    @staticmethod
    def _workspace(group: Optional[Any], tensor: Tensor) -> Optional[Any]:
        if not tensor.is_cuda or tensor.dtype not in (torch.bfloat16, torch.float32):
            return None
        if tensor.numel() == 0 or tensor.numel() * tensor.element_size() > STAGING_LIMIT_BYTES:
            return None
        return symmetric.workspace_for(group if group is not None else dist.group.WORLD)

    @staticmethod
    def _stage(ws: Any, numel: int, dtype: torch.dtype) -> Optional[Tensor]:
        """One of two symmetric staging buffers of at least ``numel`` elements (16-byte
        multiple), alternating: a rank that is one call ahead never overwrites a buffer that a
        peer of the previous call may still be reading.  Allocation is collective over the
        group (every rank asks for the same sizes in the same order) and cannot happen during
        a CUDA-graph capture: the first call of a size has to come before."""
        per = 16 // torch.empty((), dtype=dtype).element_size()
        padded = (numel + per - 1) // per * per
        cache = ws.__dict__.setdefault("_backend_stage", {})
        key = (padded, dtype)
        entry = cache.get(key)
        if entry is None:
            if torch.cuda.is_current_stream_capturing():
                return None
            bufs = [ws.alloc_tensor(padded, dtype) for _ in range(2)]
            if any(b is None for b in bufs):
                return None
            for b in bufs:
                b.zero_()
            entry = cache[key] = [bufs, 0]
        bufs, turn = entry
        entry[1] = turn ^ 1
        return bufs[turn]

    # --------------------------------------------------------- collectives --
    def all_reduce(self, tensor: Tensor, *, group: Optional[Any] = None, op: str = "sum",
                   async_op: bool = False) -> Any:
        ws = self._workspace(group, tensor) if op.lower() == "sum" and tensor.is_contiguous() else None
        buf = self._stage(ws, tensor.numel(), tensor.dtype) if ws is not None else None
        if buf is None:
            self._count("all_reduce", False)
            return super().all_reduce(tensor, group=group, op=op, async_op=async_op)
        n = tensor.numel()
        buf[:n].copy_(tensor.reshape(-1))
        if buf.numel() > n:
            buf[n:].zero_()
        ws.all_reduce_scale_(buf, 1.0, channel=CHANNEL_AUX)
        tensor.copy_(buf[:n].view_as(tensor))
        self._count("all_reduce", True)
        return _Done() if async_op else tensor

    def _gathered(self, tensor: Tensor, group: Optional[Any]) -> Optional[Tensor]:
        """``[size, numel]`` with every rank's flattened ``tensor`` or None (library path)."""
        ws = self._workspace(group, tensor)
        if ws is None or tensor.numel() * tensor.element_size() * ws.size > STAGING_LIMIT_BYTES:
            return None
        per = 16 // tensor.element_size()
        flat = tensor.reshape(-1)
        pad = (-flat.numel()) % per
        if pad:
            flat = torch.nn.functional.pad(flat, (0, pad))
        capturing = torch.cuda.is_current_stream_capturing()
        cache = ws.__dict__.get("_ag_cache", {})
        if (flat.numel() * flat.element_size(), flat.dtype) not in cache and capturing:
            return None
        if capturing:
            # A replayed graph gathers into the SAME buffer every time (the alternation of
            # the two result buffers happens on the host): make sure every rank has consumed
            # the previous replay's result before any peer stores into it again.
            ws.barrier(CHANNEL_AUX)
        return ws.all_gather(flat.contiguous())[:, : tensor.numel()]

    def all_gather_into_tensor(self, output: Tensor, input: Tensor, *, group: Optional[Any] = None) -> Tensor:
        got = self._gathered(input, group)
        if got is None:
            self._count("all_gather_into_tensor", False)
            return super().all_gather_into_tensor(output, input, group=group)
        output.copy_(got.reshape(output.shape))
        self._count("all_gather_into_tensor", True)
        return output

    def all_gather(self, tensor_list: list[Tensor], tensor: Tensor, *, group: Optional[Any] = None) -> list[Tensor]:
        got = self._gathered(tensor, group)
        if got is None:
            self._count("all_gather", False)
            return super().all_gather(tensor_list, tensor, group=group)
        for dst, row in zip(tensor_list, got):
            dst.copy_(row.view_as(dst))
        self._count("all_gather", True)
        return tensor_list

    def reduce_scatter(self, output: Tensor, input_list: list[Tensor], *, group: Optional[Any] = None,
                       op: str = "sum") -> Tensor:
        got = None
        if op.lower() == "sum" and input_list and all(t.shape == output.shape for t in input_list):
            got = self._gathered(torch.cat([t.reshape(-1) for t in input_list]), group)
        if got is None:
            self._count("reduce_scatter", False)
            return super().reduce_scatter(output, input_list, group=group, op=op)
        ws = symmetric.workspace_for(group if group is not None else dist.group.WORLD)
        n = output.numel()
        mine = got[:, ws.rank * n:(ws.rank + 1) * n]           # every rank's contribution to my shard
        output.copy_(mine.float().sum(0).view_as(output))
        self._count("reduce_scatter", True)
        return output

    def broadcast(self, tensor: Tensor, src: int, *, group: Optional[Any] = None) -> Tensor:
        got = self._gathered(tensor, group) if tensor.is_contiguous() else None
        if got is None:
            self._count("broadcast", False)
            return super().broadcast(tensor, src, group=group)
        g = group if group is not None else dist.group.WORLD
        tensor.copy_(got[dist.get_group_rank(g, src)].view_as(tensor))
        self._count("broadcast", True)
        return tensor

    def barrier(self, *, group: Optional[Any] = None) -> None:
        ws = symmetric.workspace_for(group if group is not None else dist.group.WORLD) \
            if torch.cuda.is_available() else None
        if ws is None:
            self._count("barrier", False)
            return super().barrier(group=group)
        ws.barrier(CHANNEL_AUX)
        if not torch.cuda.is_current_stream_capturing():
            torch.cuda.current_stream(ws.device).synchronize()   # torch's barrier blocks the host too
        self._count("barrier", True)
