"""Symmetric memory over CUDA IPC: buffers that every rank of a process group
can address directly, plus the signal pads the peer-memory kernels use.

A :class:`SymmetricWorkspace` belongs to one process group of GPUs on one node.
``alloc_tensor`` is a collective over that group: every rank allocates the same
number of bytes, the IPC handles are exchanged with ``all_gather_object`` and
each rank maps its peers' allocations, so a kernel can be handed the table of
all ranks' pointers (``csrc/comm.cu``).  Plain peer loads and stores only --
no multicast objects are created.

The reference has no counterpart: its only transport is ``torch.distributed``
(nano_megatron/distributed/torch_backend.py:22-80).
"""
from __future__ import annotations

import ctypes
import os
from typing import Any, Callable, Optional

import torch
import torch.distributed as dist

from ..ops import native
from . import symmetric

#: ~1 s at 1.9 GHz; a peer that never arrives ends the wait with a status code
DEFAULT_BUDGET_CYCLES = 2_000_000_000
CHANNEL_TP, CHANNEL_DP, CHANNEL_CP, CHANNEL_AUX = 0, 1, 2, 3
# Grid of the gradient-bucket all-reduce.  Negative: the overlap-first kernel
# with that many blocks (it shares SMs with the backward GEMMs instead of taking
# them over); positive: the latency-first kernel.
DDP_ALLREDUCE_BLOCKS = int(os.environ.get("NMB_DDP_AR_BLOCKS", "-148"))
# The in-switch variant moves half the bytes per GPU and issues one load and one
# store per 16 bytes, so fewer blocks keep the links busy.
DDP_MULTIMEM_BLOCKS = int(os.environ.get("NMB_DDP_MM_BLOCKS", "-64"))
# Arena: tensors up to NMB_SYMM_ARENA_MB MiB (default 256, 0 = off) are carved
# out of shared symmetric allocations of that size: one IPC handle, one handle
# exchange and, at teardown, one unmap per peer per arena instead of per tensor
# (a model has hundreds of symmetric tensors; unmapping them one by one from
# seven peers made the teardown of an 8-rank job take minutes).
ARENA_BYTES = int(os.environ.get("NMB_SYMM_ARENA_MB", "256")) << 20


class _RawCuda:
    """Exposes a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmetricAllocation:
    def __init__(self, local_ptr: int, peer_ptrs: list[int], nbytes: int, device: torch.device) -> None:
        self.local_ptr, self.peer_ptrs, self.nbytes = local_ptr, peer_ptrs, nbytes
        self.bytes = torch.as_tensor(_RawCuda(local_ptr, nbytes), device=device)

    def table(self):
        arr = (ctypes.c_void_p * len(self.peer_ptrs))()
        for i, p in enumerate(self.peer_ptrs):
            arr[i] = p
        return arr


class SymmetricWorkspace:
    def __init__(self, group: Any, *, budget_cycles: int = DEFAULT_BUDGET_CYCLES) -> None:
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.budget = int(budget_cycles)
        lib = native.lib()
        mr, mb, ch = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        lib.nmb_comm_limits(ctypes.byref(mr), ctypes.byref(mb), ctypes.byref(ch))
        self.max_ranks, self.max_blocks, self.channels = mr.value, mb.value, ch.value
        if self.size > self.max_ranks:
            raise RuntimeError(f"group of {self.size} ranks exceeds the kernel limit of {self.max_ranks}")
        self._closed = False
        self._multicast: list = []
        self._multicast_bytes = 0
        self._multicast_failed = False
        self._arena: Optional[SymmetricAllocation] = None
        self._arena_used = 0
        self._allocs: list[SymmetricAllocation] = []
        self._by_ptr: dict[int, tuple[SymmetricAllocation, int]] = {}
        self.pad = self._alloc_raw(self.channels * self.max_blocks * self.max_ranks * 4)
        self.epochs = torch.zeros(self.channels * self.max_blocks, dtype=torch.int32, device=self.device)
        self.status = native.status_word(self.device)
        dist.barrier(group=group)

    def close(self) -> None:
        """Collective, orderly release: every rank unmaps its peers' buffers, the
        group meets, then every rank frees its own.  Tensors handed out by this
        workspace must not be used afterwards."""
        if self._closed:
            return
        self._closed = True
        lib = native.lib()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)          # nobody's kernels still touch a peer buffer
        for alloc in self._allocs:
            for r, ptr in enumerate(alloc.peer_ptrs):
                if r != self.rank and ptr:
                    lib.nmb_symm_close(ctypes.c_void_p(ptr))
        dist.barrier(group=self.group)          # nobody still maps my buffers
        self._multicast.clear()
        for alloc in self._allocs:
            alloc.bytes = None
            lib.nmb_symm_free(ctypes.c_void_p(alloc.local_ptr))
        self._allocs.clear()
        self._by_ptr.clear()
        self._arena = None

    # ------------------------------------------------------------ allocation --
    def _alloc_raw(self, nbytes: int) -> SymmetricAllocation:
        nbytes = (int(nbytes) + 255) // 256 * 256
        lib = native.lib()
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        native.check_rc(lib.nmb_symm_alloc(ctypes.c_longlong(nbytes), ctypes.byref(ptr), handle), "nmb_symm_alloc")
        native.launches -= 1  # not a kernel
        mine = bytes(handle)
        everyone: list[Any] = [None] * self.size
        dist.all_gather_object(everyone, (mine, nbytes), group=self.group)
        peers: list[int] = []
        for r, (h, nb) in enumerate(everyone):
            if nb != nbytes:
                raise RuntimeError("symmetric allocation sizes differ between ranks")
            if r == self.rank:
                peers.append(ptr.value)
                continue
            remote = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            native.check_rc(lib.nmb_symm_open(buf, ctypes.byref(remote)), "nmb_symm_open")
            native.launches -= 1
            peers.append(remote.value)
        alloc = SymmetricAllocation(ptr.value, peers, nbytes, self.device)
        self._allocs.append(alloc)
        return alloc

    def alloc_tensor(self, numel: int, dtype: torch.dtype) -> Optional[torch.Tensor]:
        """Collective: a zero-filled 1-D tensor of ``numel`` elements in symmetric memory."""
        item = torch.empty((), dtype=dtype).element_size()
        nbytes = numel * item
        if 0 < nbytes <= ARENA_BYTES:
            # Every rank makes the same requests in the same order, so the offsets
            # inside the arena agree across ranks (peers_of adds the same offset).
            step = (nbytes + 1023) // 1024 * 1024
            if self._arena is None or self._arena_used + step > self._arena.nbytes:
                self._arena = self._alloc_raw(ARENA_BYTES)
                self._arena_used = 0
            alloc, off = self._arena, self._arena_used
            self._arena_used += step
        else:
            alloc, off = self._alloc_raw(nbytes), 0
        if off == 0 and nbytes == alloc.nbytes:
            t = alloc.bytes.view(dtype)
        else:
            # A tensor of its own (not a view of the arena): tensors carved from one
            # arena must not share an autograd version counter, or an in-place
            # write to one would invalidate every other one saved for backward.
            t = torch.as_tensor(_RawCuda(alloc.local_ptr + off, nbytes), device=self.device).view(dtype)
        self._by_ptr[t.data_ptr()] = (alloc, off)
        return t

    def peers_of(self, t: torch.Tensor) -> list[int]:
        """Device pointers of ``t``'s counterpart on every rank (``t`` must come from ``alloc_tensor``)."""
        for alloc in self._allocs:
            off = t.data_ptr() - alloc.local_ptr
            if 0 <= off < alloc.nbytes:
                return [p + off for p in alloc.peer_ptrs]
        raise ValueError("tensor is not in symmetric memory of this workspace")

    def peer_table(self, t: torch.Tensor):
        ptrs = self.peers_of(t)
        arr = (ctypes.c_void_p * len(ptrs))()
        for i, p in enumerate(ptrs):
            arr[i] = p
        return arr

    def contains(self, t: torch.Tensor) -> bool:
        """Whether ``t`` lives in symmetric memory of this workspace."""
        ptr = t.data_ptr()
        return any(a.local_ptr <= ptr < a.local_ptr + a.nbytes for a in self._allocs)

    def peer_strided(self, t: torch.Tensor, rank: int) -> torch.Tensor:
        """``t`` (any strided view into symmetric memory) as seen in ``rank``'s
        copy of the same allocation: same shape and strides, peer-mapped memory."""
        if rank == self.rank:
            return t
        ptr = self.peers_of(t)[rank]
        span = sum((n - 1) * st for n, st in zip(t.shape, t.stride())) + 1
        raw = torch.as_tensor(_RawCuda(ptr, span * t.element_size()), device=self.device)
        return raw.view(t.dtype).as_strided(t.shape, t.stride())

    def cp_dkv_reduce(self, stage_k: torch.Tensor, stage_v: torch.Tensor, out_k: torch.Tensor, out_v: torch.Tensor,
                      first: int, *, channel: int = CHANNEL_CP, rope=None) -> None:
        """``out_k / out_v [B, S, H, d] = sum over slots first.. of stage_k / stage_v
        [size, B, S, H, d]`` after a flag round of the group inside the same
        launch (see ``cp_dkv_reduce_kernel``); ``rope`` un-rotates dK."""
        b, s, h, d = out_k.shape
        assert out_k.stride() == out_v.stride() and out_k.stride(3) == 1
        rc = native.lib().nmb_cp_dkv_reduce(
            native.ptr(stage_k), native.ptr(stage_v), native.ptr(out_k), native.ptr(out_v),
            ctypes.c_longlong(out_k.stride(0)), ctypes.c_longlong(out_k.stride(1)), ctypes.c_longlong(out_k.stride(2)),
            ctypes.c_int(b), ctypes.c_int(s), ctypes.c_int(h), ctypes.c_int(d), ctypes.c_int(first),
            self.pad.table(), native.ptr(self.epochs), ctypes.c_int(channel), ctypes.c_int(self.rank),
            ctypes.c_int(self.size), native.ptr(rope.table if rope is not None else None),
            native.ptr(rope.positions if rope is not None else None), native.ptr(self.status),
            ctypes.c_longlong(self.budget), native.stream_ptr(self.device))
        native.check_rc(rc, "nmb_cp_dkv_reduce")

    def peer_view(self, t: torch.Tensor, rank: int) -> torch.Tensor:
        """``t``'s counterpart on ``rank`` as a tensor of this process (peer-mapped memory)."""
        if rank == self.rank:
            return t
        ptr = self.peers_of(t)[rank]
        nbytes = t.numel() * t.element_size()
        raw = torch.as_tensor(_RawCuda(ptr, nbytes), device=self.device)
        return raw.view(t.dtype).view(t.shape)

    # ------------------------------------------------------------ collectives --
    def barrier(self, channel: int = CHANNEL_AUX) -> None:
        """Device-side barrier of the group on the current stream (one tiny kernel)."""
        rc = native.lib().nmb_symm_barrier(self.pad.table(), native.ptr(self.epochs), ctypes.c_int(channel),
                                           ctypes.c_int(self.rank), ctypes.c_int(self.size), native.ptr(self.status),
                                           ctypes.c_longlong(self.budget), native.stream_ptr(self.device))
        native.check_rc(rc, "nmb_symm_barrier")

    def all_reduce_scale_(self, t: torch.Tensor, scale: float, *, channel: int = CHANNEL_DP, blocks: int = 128) -> None:
        """In-place ``t = sum_over_ranks(t) * scale`` for a tensor from ``alloc_tensor``.
        ``blocks < 0`` selects the overlap-first kernel (128 threads x at most 80
        registers per block, ``-blocks`` blocks) that fits beside a resident GEMM CTA."""
        assert t.dtype in (torch.bfloat16, torch.float32) and t.is_contiguous()
        rc = native.lib().nmb_allreduce_scale(
            self.peer_table(t), self.pad.table(), native.ptr(self.epochs), ctypes.c_int(channel),
            ctypes.c_int(self.rank), ctypes.c_int(self.size), ctypes.c_longlong(t.numel()),
            ctypes.c_int(int(t.dtype == torch.bfloat16)), ctypes.c_float(scale), ctypes.c_int(blocks),
            native.ptr(self.status), ctypes.c_longlong(self.budget), native.stream_ptr(self.device))
        native.check_rc(rc, "nmb_allreduce_scale")

    def all_gather(self, src: torch.Tensor, *, channel: int = CHANNEL_AUX) -> torch.Tensor:
        """``[size, *src.shape]`` with every rank's ``src`` (peer stores + one flag
        round; a plain kernel, so it can be captured in a CUDA graph).  The result
        lives in a cached symmetric buffer that is overwritten by the second next
        call with the same shape: consume it (or copy it) before that."""
        src = src.contiguous()
        nbytes = src.numel() * src.element_size()
        if nbytes % 16 != 0:
            raise ValueError("peer all-gather needs a multiple of 16 bytes")
        key = (nbytes, src.dtype)
        cache = self.__dict__.setdefault("_ag_cache", {})
        if key not in cache:
            cache[key] = [[self.alloc_tensor(self.size * src.numel(), src.dtype) for _ in range(2)], 0]
        bufs, turn = cache[key]
        cache[key][1] = turn ^ 1
        dst = bufs[turn]
        rc = native.lib().nmb_peer_allgather(
            native.ptr(src), self.peer_table(dst), self.pad.table(), native.ptr(self.epochs), ctypes.c_int(channel),
            ctypes.c_int(self.rank), ctypes.c_int(self.size), ctypes.c_longlong(nbytes), native.ptr(self.status),
            ctypes.c_longlong(self.budget), native.stream_ptr(self.device))
        native.check_rc(rc, "nmb_peer_allgather")
        return dst.view(self.size, *src.shape)

    def embedding_scatter(self, ids: torch.Tensor, positions: Optional[torch.Tensor], tok_w: torch.Tensor,
                          pos_w: Optional[torch.Tensor], out: torch.Tensor, vocab_start: int, seq_len: int,
                          *, to_all: bool = False) -> None:
        """Every token row owned by this rank's vocabulary shard is written (token +
        position embedding) into the sequence-shard owner's ``out`` (symmetric,
        ``[B * S/size, H]``) or, with ``to_all``, into every rank's ``out``
        (``[B * S, H]``)."""
        n_tokens = ids.numel()
        rc = native.lib().nmb_embedding_scatter(
            native.ptr(ids), native.ptr(positions), native.ptr(tok_w), native.ptr(pos_w), self.peer_table(out),
            ctypes.c_int(self.size), ctypes.c_int(n_tokens), ctypes.c_int(tok_w.shape[1]), ctypes.c_int(vocab_start),
            ctypes.c_int(tok_w.shape[0]), ctypes.c_int(seq_len), ctypes.c_int(max(seq_len // self.size, 1)),
            ctypes.c_int(int(to_all)), native.stream_ptr(self.device))
        native.check_rc(rc, "nmb_embedding_scatter")

    # ------------------------------------------------------------- multimem --
    def alloc_multicast(self, numel: int, dtype: torch.dtype) -> Optional[tuple[torch.Tensor, int]]:
        """Collective: a zero-filled tensor that is also mapped at an NVSwitch
        multicast address on every rank of the group, for in-switch reductions
        (``multimem.ld_reduce`` / ``multimem.st``).  Allocation and handle
        exchange are ``torch.distributed``'s symmetric memory (the multicast
        object needs the driver's virtual-memory API and a file-descriptor
        exchange between the processes); the kernels that use the address are
        this package's.  Returns ``(tensor, multicast pointer)``, or ``None``
        when multicast is not available (switched off with ``NMB_MULTIMEM=0``,
        no NVSwitch support, a group this rendezvous cannot serve): the caller
        then uses plain peer memory."""
        if os.environ.get("NMB_MULTIMEM", "1") == "0" or self._multicast_failed:
            return None
        try:
            import torch.distributed._symmetric_memory as tsm
            t = tsm.empty(numel, dtype=dtype, device=self.device)
            handle = tsm.rendezvous(t, self.group)
            mc = int(handle.multicast_ptr)
        except Exception:
            mc = 0
        # every rank must take the same path
        flag = torch.tensor([1 if mc else 0], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self._multicast_failed = True
            return None
        t.zero_()
        self._multicast.append((t, handle))
        self._multicast_bytes += t.numel() * t.element_size()
        return t, mc

    def multimem_all_reduce_scale_(self, mc: int, numel: int, is_bf16: bool, scale: float, *,
                                   channel: int = CHANNEL_DP, blocks: int = 64) -> None:
        """In-place ``sum_over_ranks * scale`` of the buffer mapped at multicast
        address ``mc`` (from :meth:`alloc_multicast`), reduced inside the switch."""
        rc = native.lib().nmb_multimem_allreduce_scale(
            ctypes.c_void_p(mc), self.pad.table(), native.ptr(self.epochs), ctypes.c_int(channel),
            ctypes.c_int(self.rank), ctypes.c_int(self.size), ctypes.c_longlong(numel), ctypes.c_int(int(is_bf16)),
            ctypes.c_float(scale), ctypes.c_int(blocks), native.ptr(self.status), ctypes.c_longlong(self.budget),
            native.stream_ptr(self.device))
        native.check_rc(rc, "nmb_multimem_allreduce_scale")

    def make_multimem_allreduce_mean(self, flat: torch.Tensor, mc: int) -> Callable[[torch.Tensor, int], bool]:
        """Reducer for a DDP bucket whose gradients live at the start of ``flat``
        (a multicast-mapped tensor padded to 16 bytes)."""
        per = 8 if flat.dtype == torch.bfloat16 else 4
        if flat.numel() % per != 0:
            raise ValueError("bucket buffer must be padded to a multiple of 16 bytes")
        numel, is_bf16 = flat.numel(), flat.dtype == torch.bfloat16

        def reduce(buf: torch.Tensor, divisor: int) -> bool:
            if buf.data_ptr() != flat.data_ptr() or buf.numel() > numel:
                return False
            self.multimem_all_reduce_scale_(mc, numel, is_bf16, 1.0 / divisor, blocks=DDP_MULTIMEM_BLOCKS)
            return True

        return reduce

    def allocated_bytes(self) -> int:
        """Device memory held by this workspace on this rank."""
        return sum(a.nbytes for a in self._allocs) + self._multicast_bytes

    def make_allreduce_mean(self, flat: torch.Tensor) -> Callable[[torch.Tensor, int], bool]:
        """Reducer for a DDP bucket whose gradients live at the start of ``flat``
        (see ``GradBucket.fused_reduce``).  ``flat`` is the whole symmetric
        allocation, padded to a multiple of 16 bytes, so every bucket size can
        be reduced by the kernel and no call falls back to the library path."""
        per = 8 if flat.dtype == torch.bfloat16 else 4
        if flat.numel() % per != 0:
            raise ValueError("bucket buffer must be padded to a multiple of 16 bytes")
        table, pads = self.peer_table(flat), self.pad.table()
        numel, is_bf16 = flat.numel(), int(flat.dtype == torch.bfloat16)

        def reduce(buf: torch.Tensor, divisor: int) -> bool:
            if buf.data_ptr() != flat.data_ptr() or buf.numel() > numel:
                return False
            rc = native.lib().nmb_allreduce_scale(
                table, pads, native.ptr(self.epochs), ctypes.c_int(CHANNEL_DP), ctypes.c_int(self.rank),
                ctypes.c_int(self.size), ctypes.c_longlong(numel), ctypes.c_int(is_bf16),
                ctypes.c_float(1.0 / divisor), ctypes.c_int(DDP_ALLREDUCE_BLOCKS), native.ptr(self.status),
                ctypes.c_longlong(self.budget), native.stream_ptr(self.device))
            native.check_rc(rc, "nmb_allreduce_scale")
            return True

        return reduce


def enable_symmetric_memory(ctx: Any) -> dict[str, SymmetricWorkspace]:
    """Create and register workspaces for the TP, CP and DP x CP groups of ``ctx``
    (those with more than one rank).  Collective over the whole job."""
    made: dict[str, SymmetricWorkspace] = {}
    for name, group, size in (
        ("tp", ctx.tensor_parallel_group, ctx.tensor_parallel_size),
        ("cp", ctx.context_parallel_group, ctx.context_parallel_size),
        ("dp-cp", ctx.data_context_parallel_group, ctx.data_parallel_size * ctx.context_parallel_size),
    ):
        if size > 1 and symmetric.workspace_for(group) is None:
            ws = SymmetricWorkspace(group)
            symmetric.register_workspace(group, ws)
            made[name] = ws
    from ..ops import fused_tp
    fused_tp.ENABLED = True
    return made
