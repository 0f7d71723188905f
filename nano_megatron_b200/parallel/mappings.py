"""Tensor-parallel and sequence-parallel operators and the column / row linears.

Public names and semantics follow the reference
(nano_megatron/parallel/mappings.py:32-463): the conjugate pair
copy-to-TP (identity / all-reduce) and reduce-from-TP (all-reduce / identity),
the three sequence-parallel region functions on dim 1 of ``[B, S, ...]``, the
shard helpers, and ``ColumnParallelLinear`` / ``RowParallelLinear`` built from a
*full* weight.  The matmuls run on the tcgen05 GEMM with fused bias / GELU /
residual epilogues when the tensors are bf16 on a GPU, and gradients of
sequence-parallel replicated parameters are reduced with ONE coalesced
all-reduce per backward pass instead of one blocking all-reduce per parameter
(reference: :166-187).
"""
from __future__ import annotations

import weakref
from typing import Any, Optional

import torch
import torch.nn as nn
from torch import Tensor

from ..distributed.backend import CommBackend
from ..ops import functional as OF

SEQ_DIM = 1


def _require_seq_tensor(x: Tensor) -> None:
    if x.dim() < 2:
        raise ValueError(f"sequence-parallel tensor must have dim >= 2 (layout [B, S, ...]), got dim={x.dim()}")


def _require_divisible(seq_len: int, tp_size: int) -> None:
    if tp_size < 1:
        raise ValueError(f"tp_size must be >= 1, got {tp_size}")
    if seq_len % tp_size != 0:
        raise ValueError(f"sequence length ({seq_len}) not divisible by tp_size ({tp_size})")


def _wait(work: Any) -> None:
    if hasattr(work, "wait"):
        work.wait()


class CommunicationBuffer:
    """Cache of communication buffers keyed by (shape, dtype, device)."""

    def __init__(self) -> None:
        self._buffers: dict[tuple[tuple[int, ...], torch.dtype, torch.device], Tensor] = {}

    def get_buffer(self, shape: tuple[int, ...], dtype: torch.dtype, device: torch.device) -> Tensor:
        key = (tuple(shape), dtype, torch.device(device))
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.empty(tuple(shape), dtype=dtype, device=device)
            self._buffers[key] = buf
        return buf


# ----------------------------------------------- sequence <-> full gathers --
def _all_gather_seq(x: Tensor, group: Any, backend: CommBackend, tp_size: int) -> Tensor:
    """Concatenate the ranks' ``[B, S/t, ...]`` shards along dim 1 with one
    single-buffer all-gather (no list API, no ``torch.cat``)."""
    x = x.contiguous()
    stacked = x.new_empty((tp_size, *x.shape))
    # (concatenation along dim 0 is the layout every backend accepts)
    backend.all_gather_into_tensor(stacked.view(tp_size * x.shape[0], *x.shape[1:]), x, group=group)
    if x.shape[0] == 1:
        return stacked.view(1, tp_size * x.shape[1], *x.shape[2:])
    return stacked.transpose(0, 1).reshape(x.shape[0], tp_size * x.shape[1], *x.shape[2:])


def _reduce_scatter_seq(x: Tensor, group: Any, backend: CommBackend, tp_size: int) -> Tensor:
    _require_divisible(x.size(SEQ_DIM), tp_size)
    pieces = [c.contiguous() for c in x.chunk(tp_size, dim=SEQ_DIM)]
    out = torch.empty_like(pieces[0])
    backend.reduce_scatter(out, pieces, group=group, op="sum")
    return out


class _ScatterToSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: Tensor, group: Any, backend: CommBackend, tp_rank: int, tp_size: int) -> Tensor:
        ctx.comm = (group, backend, tp_rank, tp_size)
        if tp_size == 1:
            return x
        _require_seq_tensor(x)
        _require_divisible(x.size(SEQ_DIM), tp_size)
        width = x.size(SEQ_DIM) // tp_size
        return x.narrow(SEQ_DIM, tp_rank * width, width).contiguous()

    @staticmethod
    def backward(ctx: Any, grad: Tensor):
        group, backend, _, tp_size = ctx.comm
        if tp_size == 1:
            return grad, None, None, None, None
        return _all_gather_seq(grad, group, backend, tp_size), None, None, None, None


class _GatherFromSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: Tensor, group: Any, backend: CommBackend, tp_rank: int, tp_size: int) -> Tensor:
        ctx.comm = (group, backend, tp_rank, tp_size)
        if tp_size == 1:
            return x
        _require_seq_tensor(x)
        return _all_gather_seq(x, group, backend, tp_size)

    @staticmethod
    def backward(ctx: Any, grad: Tensor):
        group, backend, _, tp_size = ctx.comm
        if tp_size == 1:
            return grad, None, None, None, None
        return _reduce_scatter_seq(grad, group, backend, tp_size), None, None, None, None


class _ReduceScatterToSequenceParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: Tensor, group: Any, backend: CommBackend, tp_rank: int, tp_size: int) -> Tensor:
        ctx.comm = (group, backend, tp_rank, tp_size)
        if tp_size == 1:
            return x
        _require_seq_tensor(x)
        return _reduce_scatter_seq(x, group, backend, tp_size)

    @staticmethod
    def backward(ctx: Any, grad: Tensor):
        group, backend, _, tp_size = ctx.comm
        if tp_size == 1:
            return grad, None, None, None, None
        return _all_gather_seq(grad, group, backend, tp_size), None, None, None, None


def scatter_to_sequence_parallel_region(x: Tensor, group: Any, backend: CommBackend, tp_rank: int, tp_size: int) -> Tensor:
    return _ScatterToSequenceParallelRegion.apply(x, group, backend, tp_rank, tp_size)


def gather_from_sequence_parallel_region(x: Tensor, group: Any, backend: CommBackend, tp_rank: int, tp_size: int) -> Tensor:
    return _GatherFromSequenceParallelRegion.apply(x, group, backend, tp_rank, tp_size)


def reduce_scatter_to_sequence_parallel_region(x: Tensor, group: Any, backend: CommBackend, tp_rank: int, tp_size: int) -> Tensor:
    return _ReduceScatterToSequenceParallelRegion.apply(x, group, backend, tp_rank, tp_size)


# ------------------------------- replicated-parameter gradients under SP --
class _SPGradReducer:
    """Coalesces the TP all-reduce of sequence-parallel replicated-parameter grads.

    With SP, LayerNorm weights/biases and the row-parallel bias see only this
    rank's ``S/t`` tokens, so their gradients are partial sums.  Each parameter's
    hook records the incoming gradient; a callback queued on the autograd engine
    runs once at the end of the backward pass, all-reduces all recorded
    gradients in one flat buffer and adds the other ranks' share to ``.grad``
    (correct under gradient accumulation, since only this pass's gradients are
    exchanged).
    """

    _instances: "weakref.WeakValueDictionary[tuple[int, int], _SPGradReducer]" = weakref.WeakValueDictionary()

    def __init__(self, group: Any, backend: CommBackend) -> None:
        self.group, self.backend = group, backend
        self._pending: list[tuple[nn.Parameter, Tensor]] = []
        self._queued = False

    @classmethod
    def for_group(cls, group: Any, backend: CommBackend) -> "_SPGradReducer":
        key = (id(group), id(backend))
        inst = cls._instances.get(key)
        if inst is None or inst.group is not group:
            inst = cls(group, backend)
            cls._instances[key] = inst
        return inst

    def attach(self, param: nn.Parameter) -> None:
        param._nmb_sp_replicated = True  # DDP syncs these after the TP reduction
        param._nmb_sp_reducer = self     # keeps the reducer alive with the parameter

        def hook(grad: Tensor) -> Tensor:
            self._pending.append((param, grad))
            if not self._queued:
                self._queued = True
                torch.autograd.Variable._execution_engine.queue_callback(self.flush)
            return grad

        param.register_hook(hook)

    def flush(self) -> None:
        pending, self._pending, self._queued = self._pending, [], False
        if not pending:
            return
        by_dtype: dict[torch.dtype, list[tuple[nn.Parameter, Tensor]]] = {}
        for item in pending:
            by_dtype.setdefault(item[1].dtype, []).append(item)
        for items in by_dtype.values():
            local = torch.cat([g.reshape(-1) for _, g in items])
            ws = None
            if local.is_cuda:
                from ..distributed import symmetric
                ws = symmetric.workspace_for(self.group)
            if ws is not None:
                pad = (-local.numel()) % 8
                padded = torch.nn.functional.pad(local, (0, pad)) if pad else local
                everyone = ws.all_gather(padded)            # [ranks, n]; peer stores, no NCCL
                total = everyone.float().sum(0)[: local.numel()].to(local.dtype)
            else:
                total = local.clone()
                _wait(self.backend.all_reduce(total, group=self.group, op="sum", async_op=True))
            remote = total - local
            offset = 0
            for p, g in items:
                n = g.numel()
                target = getattr(p, "main_grad", None)
                if target is None:
                    target = p.grad
                if target is not None:
                    target.add_(remote[offset:offset + n].view_as(target))
                offset += n


def register_sequence_parallel_grad_allreduce(param: nn.Parameter, group: Any, backend: CommBackend) -> None:
    """Sum the gradient of a replicated parameter that only saw a sequence shard."""
    if not param.requires_grad:
        return
    _SPGradReducer.for_group(group, backend).attach(param)


# ------------------------------------------------------ TP conjugate pair --
class _CopyToTPRegion(torch.autograd.Function):
    """Forward identity on a replicated input; backward sums the partial input grads."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, group: Any, backend: CommBackend,
                buffer_manager: Optional[CommunicationBuffer] = None) -> Tensor:
        ctx.comm = (group, backend, buffer_manager)
        return x

    @staticmethod
    def backward(ctx: Any, grad: Tensor):
        group, backend, buffers = ctx.comm
        if buffers is not None:
            buf = buffers.get_buffer(grad.shape, grad.dtype, grad.device)
            buf.copy_(grad)
            grad = buf
        elif not grad.is_contiguous():
            grad = grad.contiguous()   # e.g. an expanded gradient: the collective writes in place
        _wait(backend.all_reduce(grad, group=group, op="sum", async_op=True))
        return grad, None, None, None


class _ReduceFromTPRegion(torch.autograd.Function):
    """Forward sums the ranks' partial results; backward identity."""

    @staticmethod
    def forward(ctx: Any, x: Tensor, group: Any, backend: CommBackend,
                buffer_manager: Optional[CommunicationBuffer] = None) -> Tensor:
        if buffer_manager is not None:
            buf = buffer_manager.get_buffer(x.shape, x.dtype, x.device)
            buf.copy_(x)
            x = buf
        elif not (x.is_leaf and x.requires_grad):
            # reduced in place and handed back: tell autograd (a leaf that requires grad
            # cannot be marked; it is returned as it is, like the reference does)
            ctx.mark_dirty(x)
        _wait(backend.all_reduce(x, group=group, op="sum", async_op=True))
        return x

    @staticmethod
    def backward(ctx: Any, grad: Tensor):
        return grad, None, None, None


# ------------------------------------------------------------ shard helpers --
def column_shard(weight: Tensor, bias: Optional[Tensor], tp_rank: int, tp_size: int):
    rows = weight.shape[0]
    if rows % tp_size != 0:
        raise ValueError(f"column output dim ({rows}) not divisible by tp_size ({tp_size})")
    n = rows // tp_size
    sl = slice(tp_rank * n, (tp_rank + 1) * n)
    return weight.data[sl, :].clone(), (bias.data[sl].clone() if bias is not None else None)


def blockwise_column_shard(weight: Tensor, bias: Optional[Tensor], tp_rank: int, tp_size: int,
                           block_sizes: tuple[int, ...]):
    """Shard each logical row block (``[Q;K;V]``, ``[gate;up]``) separately so the
    local rows stay ``[block0_r; block1_r; ...]``."""
    if weight.shape[0] != sum(block_sizes):
        raise ValueError(f"column out dim ({weight.shape[0]}) != sum(block_sizes) ({sum(block_sizes)})")
    for i, size in enumerate(block_sizes):
        if size % tp_size != 0:
            raise ValueError(f"block_sizes[{i}] ({size}) not divisible by tp_size ({tp_size})")
    index, start = [], 0
    for size in block_sizes:
        n = size // tp_size
        index.append(torch.arange(start + tp_rank * n, start + (tp_rank + 1) * n))
        start += size
    rows = torch.cat(index).to(weight.device)
    return weight.data.index_select(0, rows).clone(), (bias.data.index_select(0, rows).clone() if bias is not None else None)


def fused_qkv_column_shard(weight: Tensor, bias: Optional[Tensor], tp_rank: int, tp_size: int, q_dim: int, kv_dim: int):
    return blockwise_column_shard(weight, bias, tp_rank, tp_size, (q_dim, kv_dim, kv_dim))


def row_shard(weight: Tensor, bias: Optional[Tensor], tp_rank: int, tp_size: int):
    cols = weight.shape[1]
    if cols % tp_size != 0:
        raise ValueError(f"row input dim ({cols}) not divisible by tp_size ({tp_size})")
    n = cols // tp_size
    return weight.data[:, tp_rank * n:(tp_rank + 1) * n].clone(), (bias.data.clone() if bias is not None else None)


# ---------------------------------------------------------------- linears --
class ColumnParallelLinear(nn.Module):
    """Output features sharded over the TP group; the output is never gathered."""

    def __init__(self, weight: Tensor, bias: Optional[Tensor], tp_rank: int, tp_size: int, group: Any,
                 backend: CommBackend, *, weight_is_local: bool = False, sequence_parallel: bool = False) -> None:
        super().__init__()
        if weight_is_local:
            w, b = weight.data.clone(), (bias.data.clone() if bias is not None else None)
        else:
            w, b = column_shard(weight, bias, tp_rank, tp_size)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(b) if b is not None else None
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.group, self.backend = group, backend
        self.buffer_manager = CommunicationBuffer()
        self.sequence_parallel = sequence_parallel

    def forward(self, x: Tensor, *, gelu: bool = False, split_gelu: bool = False, split_act: Optional[str] = None,
                rope: Any = None, out: Optional[Tensor] = None):
        """``split_act`` (``"gelu"`` / ``"swiglu"``; ``split_gelu=True`` means ``"gelu"``)
        returns ``(pre_activation, act(pre_activation))`` from one GEMM so that
        the following row-parallel linear can fold the activation's backward
        into its dgrad GEMM (bf16 GPU path only).  ``rope`` (a
        :class:`~nano_megatron_b200.ops.gemm.RopeSpec`, bf16 GPU path only)
        rotates the leading q / k columns of the output in the GEMM epilogue.
        ``out`` (``tp_size == 1``, bf16 GPU path) is the tensor the GEMM writes
        its result into, e.g. symmetric memory that other ranks read in place."""
        if out is not None and (self.tp_size > 1 or split_act or gelu):
            raise ValueError("an output buffer is supported for a plain projection at tp_size == 1")
        if split_gelu and split_act is None:
            split_act = "gelu"
        native = OF.native_linear_ok(x, self.weight)
        if (split_act == "swiglu" or rope is not None) and not native:
            raise ValueError("the fused SwiGLU / rotary epilogues need bf16 CUDA tensors")
        want_act = split_act or ("gelu" if gelu else None)
        if self.sequence_parallel and self.tp_size > 1 and x.dim() == 3 and native:
            from ..ops import fused_tp
            st = fused_tp.tp_fused_for(self.group) if fused_tp.ENABLED else None
            seq_len = x.shape[1] * self.tp_size
            if st is not None and st.supported(x.shape[0] * seq_len, seq_len, self.weight.shape[0]):
                # all-gather fused into the GEMM (one launch, peers' shards pulled tile by tile)
                out = fused_tp._SPColumnLinearFn.apply(x, self.weight, self.bias, st, seq_len, self, want_act, rope)
                if split_act:
                    return out
                return out[1] if gelu else out
        if not self.sequence_parallel and self.tp_size > 1 and native:
            from ..ops import fused_tp
            st = fused_tp.tp_fused_for(self.group) if fused_tp.ENABLED else None
            rows = x.numel() // x.shape[-1]
            if st is not None and st.all_reduce_supported(rows, x.shape[-1]):
                # local GEMM; the all-reduce of the input gradient rides in the dgrad GEMM
                out = fused_tp._TPColumnLinearFn.apply(x, self.weight, self.bias, st, want_act, rope)
                if split_act:
                    return out
                return out[1] if gelu else out
        if self.sequence_parallel:
            x = gather_from_sequence_parallel_region(x, self.group, self.backend, self.tp_rank, self.tp_size)
        elif self.tp_size > 1:
            x = _CopyToTPRegion.apply(x, self.group, self.backend, self.buffer_manager)
        if split_act:
            if OF.native_linear_ok(x, self.weight):
                return OF.linear_act_split(x, self.weight, self.bias, split_act)
            return None, OF.linear(x, self.weight, self.bias, gelu=True)
        return OF.linear(x, self.weight, self.bias, gelu=gelu, rope=rope, out=out)


class RowParallelLinear(nn.Module):
    """Input features sharded over the TP group; partial outputs are summed
    (all-reduce, or reduce-scatter under SP) and the replicated bias is added
    after the collective."""

    def __init__(self, weight: Tensor, bias: Optional[Tensor], tp_rank: int, tp_size: int, group: Any,
                 backend: CommBackend, *, sequence_parallel: bool = False) -> None:
        super().__init__()
        w, b = row_shard(weight, bias, tp_rank, tp_size)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(b) if b is not None else None
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.group, self.backend = group, backend
        self.buffer_manager = CommunicationBuffer()
        self.sequence_parallel = sequence_parallel
        if sequence_parallel and self.bias is not None:
            register_sequence_parallel_grad_allreduce(self.bias, group, backend)

    def forward(self, x: Tensor, *, residual: Optional[Tensor] = None, gelu_pre: Optional[Tensor] = None,
                act_pre: Optional[Tensor] = None, act: str = "gelu") -> Tensor:
        """``act_pre``: ``x`` is ``act(act_pre)`` (from ``split_act``; ``gelu_pre`` is
        the same for ``act="gelu"``); the backward then returns the gradient of
        ``act_pre``."""
        if gelu_pre is not None and act_pre is None:
            act_pre, act = gelu_pre, "gelu"
        fused = act_pre is not None and OF.native_linear_ok(x, self.weight)
        if act_pre is not None and not fused:
            raise ValueError("act_pre needs the bf16 CUDA path")
        if self.tp_size == 1:
            # Nothing to reduce: bias and residual ride in the GEMM epilogue.
            if fused:
                return OF.linear_from_act(act_pre, x, self.weight, self.bias, residual, act)
            return OF.linear(x, self.weight, self.bias, residual=residual)
        if self.sequence_parallel and x.dim() == 3 and OF.native_linear_ok(x, self.weight):
            from ..ops import fused_tp
            st = fused_tp.tp_fused_for(self.group) if fused_tp.ENABLED else None
            if st is not None and st.supported(x.shape[0] * x.shape[1], x.shape[1], self.weight.shape[0]):
                # GEMM with the reduce-scatter (and bias / residual) fused in
                return fused_tp._SPRowLinearFn.apply(x, self.weight, self.bias, residual,
                                                     act_pre if fused else None, st, x.shape[1], act)
        if not self.sequence_parallel and OF.native_linear_ok(x, self.weight):
            from ..ops import fused_tp
            st = fused_tp.tp_fused_for(self.group) if fused_tp.ENABLED else None
            rows = x.numel() // x.shape[-1]
            if st is not None and st.all_reduce_supported(rows, self.weight.shape[0]):
                # GEMM with the all-reduce (and bias / residual) fused in
                return fused_tp._TPRowLinearFn.apply(x, self.weight, self.bias, residual,
                                                     act_pre if fused else None, st, act)
        out = OF.linear_from_act(act_pre, x, self.weight, None, None, act) if fused else OF.linear(x, self.weight, None)
        if self.sequence_parallel:
            out = reduce_scatter_to_sequence_parallel_region(out, self.group, self.backend, self.tp_rank, self.tp_size)
        else:
            out = _ReduceFromTPRegion.apply(out, self.group, self.backend, self.buffer_manager)
        if self.bias is not None:
            out = out + self.bias
        if residual is not None:
            out = residual + out
        return out
