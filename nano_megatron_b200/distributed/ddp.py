"""Data-parallel wrapper with gradient buckets overlapped with backward.

Public contract as in the reference (nano_megatron/distributed/ddp.py:17-189):
gradients are averaged over the DP x CP group (divisor ``dp * cp``), parameters
are broadcast from the group's leader at construction, a bucket is reduced as
soon as all of its parameters have their gradient, ``no_sync()`` defers
everything and ``finish_grad_sync()`` (idempotent) flushes what is left.

B200-first differences:

* gradients live in persistent flat bucket buffers (``.grad`` / ``main_grad``
  are views), so a bucket is reduced in place -- no flatten / divide /
  unflatten passes -- and the weight-gradient GEMMs write into the buffers
  directly;
* on a GPU each bucket's reduction is issued on a side stream as soon as the
  bucket is complete, so it runs under the rest of the backward pass (the
  reference's per-bucket all-reduce blocks the compute stream,
  nano_megatron/distributed/bucket.py:93); ``finish_grad_sync`` joins the
  streams;
* when the buffers are in symmetric memory the reduction is one kernel that
  sums, scales by ``1/(dp*cp)`` and writes the result instead of NCCL +
  ``div_``: in the NVSwitch (``multimem.ld_reduce`` / ``multimem.st``) where the
  machine offers multicast memory, else by reading every peer's bucket over
  NVLink (``distributed/symm_mem.py``); the side stream has high priority so
  that the reduction's few blocks are scheduled beside the compute kernels;
* with ``overwrite_first_grad`` (what ``Trainer`` asks for) ``zero_grad`` stops
  zeroing the buffers of parameters whose first gradient write of a step can
  store instead of add; ``after_bucket_sync`` is a hook a trainer may use to act
  on a bucket the moment it is reduced; ``close()`` detaches the wrapper;
* the construction-time broadcast is one coalesced broadcast per dtype, not one
  per parameter (reference :85-96);
* parameters replicated under sequence parallelism (their TP reduction runs at
  the end of the backward pass) are kept in buckets that are only reduced in
  ``finish_grad_sync``.
"""
from __future__ import annotations

import weakref
from contextlib import contextmanager
from typing import TYPE_CHECKING, Any, Iterator, Optional

import torch
import torch.nn as nn

from .backend import CommBackend
from .bucket import GradBucket, build_buckets

if TYPE_CHECKING:
    from ..parallel.context import ParallelContext


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, ctx: "ParallelContext", *, bucket_cap_mb: float = 25.0,
                 broadcast_buffers: bool = False, persistent_grads: Optional[bool] = None,
                 overlap: Optional[bool] = None, overwrite_first_grad: bool = False) -> None:
        super().__init__()
        _ = broadcast_buffers  # reserved, as in the reference
        self.add_module("module", module)
        self._ctx = ctx
        self._backend: CommBackend = ctx.backend
        self._dp_group = ctx.data_context_parallel_group
        self._mean_divisor = ctx.data_parallel_size * ctx.context_parallel_size
        self._sync_group_size = self._mean_divisor
        self._bucket_cap_mb = bucket_cap_mb

        all_buckets = build_buckets(module, bucket_cap_mb)
        eager, deferred = [], []
        for b in all_buckets:
            now = [p for p in b.params if not getattr(p, "_nmb_sp_replicated", False)]
            late = [p for p in b.params if getattr(p, "_nmb_sp_replicated", False)]
            if now:
                eager.append(GradBucket(now))
            if late:
                deferred.append(GradBucket(late))
        self._buckets: list[GradBucket] = eager + deferred
        self._deferred = {id(b) for b in deferred}
        self._param_to_bucket: dict[nn.Parameter, GradBucket] = {p: b for b in self._buckets for p in b.params}
        self._param_names = {id(p): n for n, p in module.named_parameters()}
        self._hook_handles: list[Any] = []
        self._sync_done = True
        self._require_backward_grad_sync = True
        self._write_counts: dict[int, int] = {}

        device = self._param_device()
        self._on_gpu = device.type == "cuda"
        self._persistent = self._on_gpu if persistent_grads is None else bool(persistent_grads)
        self._overlap = self._on_gpu if overlap is None else bool(overlap and self._on_gpu)
        # High priority: a bucket reduction is a few dozen blocks that must become resident
        # beside whatever the compute stream is running.  At default priority the reduction of
        # the last bucket waited behind the 16 k blocks of the optimizer kernel it was meant to
        # overlap (373 us exposed per step at two ranks); kernel nodes keep the priority under
        # CUDA-graph capture.
        self._side_stream = torch.cuda.Stream(device=device, priority=-1) if self._overlap else None
        self._side_used = False
        self._flat_buffers: list[torch.Tensor] = []
        #: Called with a bucket right after its reduction has been issued, on the stream the
        #: reduction runs on (so work launched from the callback is ordered after it).  The
        #: trainer uses it to update a bucket's parameters while backward is still running.
        self.after_bucket_sync: Optional[Any] = None
        # "first write of a step overwrites" (see zero_grad): off | learning | on
        self._overwrite_first = bool(overwrite_first_grad)
        self._grad_trace: Optional[dict[int, str]] = None
        self._zero_plan: Optional[tuple[list[tuple[int, int, int]], list[nn.Parameter]]] = None
        #: buckets in the order their reduction was issued on the side stream this step, and an event after each
        self._issued: list[GradBucket] = []
        self._bucket_events: dict[int, torch.cuda.Event] = {}

        self._broadcast_params()
        if self._persistent:
            self._allocate_persistent()
        self._register_grad_hooks()

    # ---------------------------------------------------------------- set-up --
    def _param_device(self) -> torch.device:
        for p in self.module.parameters():
            return p.device
        return torch.device("cpu")

    def _broadcast_params(self) -> None:
        if self._sync_group_size == 1 or not self._param_to_bucket:
            return
        device = self._param_device()
        leader_here = self._ctx.data_parallel_rank == 0 and self._ctx.context_parallel_rank == 0
        leader = torch.tensor([self._ctx.rank if leader_here else -1], dtype=torch.long, device=device)
        self._backend.all_reduce(leader, group=self._dp_group, op="max")
        src = int(leader.item())
        by_dtype: dict[torch.dtype, list[nn.Parameter]] = {}
        for p in self._param_to_bucket:
            by_dtype.setdefault(p.dtype, []).append(p)
        for params in by_dtype.values():
            flat = torch.cat([p.data.reshape(-1) for p in params])
            self._backend.broadcast(flat, src=src, group=self._dp_group)
            offset = 0
            for p in params:
                p.data.copy_(flat[offset:offset + p.numel()].view_as(p))
                offset += p.numel()

    def _allocate_persistent(self) -> None:
        from . import symmetric

        ws = symmetric.workspace_for(self._dp_group) if self._on_gpu else None
        for b in self._buckets:
            dtype, device = b.params[0].dtype, b.params[0].device
            flat = None
            if ws is not None and self._sync_group_size > 1:
                # padded to whole 16-byte vectors so the peer kernel takes every bucket
                per = 16 // torch.empty((), dtype=dtype).element_size()
                padded_numel = (b.numel() + per - 1) // per * per
                mapped = ws.alloc_multicast(padded_numel, dtype)
                if mapped is not None:
                    # reduced inside the NVSwitch (multimem), each element crosses the links once
                    padded, mc = mapped
                    b.fused_reduce = ws.make_multimem_allreduce_mean(padded, mc)
                    flat = padded[: b.numel()]
                else:
                    padded = ws.alloc_tensor(padded_numel, dtype)
                    if padded is not None:
                        padded.zero_()
                        b.fused_reduce = ws.make_allreduce_mean(padded)
                        flat = padded[: b.numel()]
            if flat is None:
                flat = torch.zeros(b.numel(), dtype=dtype, device=device)
            b.bind_persistent(flat)
            self._flat_buffers.append(flat)

    def _register_grad_hooks(self) -> None:
        for param in self._param_to_bucket:
            self._hook_handles.append(
                param.register_post_accumulate_grad_hook(lambda _p, param=param: self._on_autograd_write(param)))
            # Kernels that accumulate into ``main_grad`` announce it here.
            param._nmb_grad_ready = (lambda param=param: self._on_direct_write(param))

    def close(self) -> None:
        """Detach from the wrapped module: remove the gradient hooks and the per-parameter
        callbacks.  The hooks are held by the parameters' autograd metadata and refer back to
        this wrapper, a cycle the garbage collector cannot see through, so a wrapper that is
        merely dropped keeps its module, gradient buffers and itself alive."""
        for handle in self._hook_handles:
            handle.remove()
        self._hook_handles = []
        for param in self._param_to_bucket:
            for attr in ("_nmb_grad_ready", "_nmb_overwrite_next"):
                if hasattr(param, attr):
                    delattr(param, attr)
        self.after_bucket_sync = None
        if self._grad_trace is not None:
            from ..ops import functional as F
            trace, self._grad_trace = self._grad_trace, None
            F._GRAD_TRACES[:] = [t for t in F._GRAD_TRACES if t is not trace]

    # ----------------------------------------------------------------- hooks --
    @contextmanager
    def no_sync(self) -> Iterator[None]:
        """Gradients still accumulate; no bucket is marked or reduced."""
        prev = self._require_backward_grad_sync
        self._require_backward_grad_sync = False
        try:
            yield
        finally:
            self._require_backward_grad_sync = prev

    def _on_autograd_write(self, param: nn.Parameter) -> None:
        # autograd added a gradient to ``.grad``: an adding write as far as the zero plan goes
        if self._grad_trace is not None:
            self._grad_trace.setdefault(id(param), "other")
        self._on_param_grad_ready(param)

    def _on_direct_write(self, param: nn.Parameter) -> None:
        if not self._require_backward_grad_sync:
            self._sync_done = False
            return
        uses = int(getattr(param, "_nmb_grad_uses", 1))
        if uses > 1:
            seen = self._write_counts.get(id(param), 0) + 1
            if seen < uses:
                self._write_counts[id(param)] = seen
                self._sync_done = False
                return
            self._write_counts[id(param)] = 0
        self._on_param_grad_ready(param)

    def _on_param_grad_ready(self, param: nn.Parameter) -> None:
        bucket = self._param_to_bucket.get(param)
        if bucket is None:
            return
        self._sync_done = False
        if not self._require_backward_grad_sync:
            return
        if bucket.mark_ready(param) and id(bucket) not in self._deferred:
            self._sync_bucket(bucket)

    def _sync_bucket(self, bucket: GradBucket) -> None:
        if self._side_stream is not None and self._sync_group_size > 1:
            self._side_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._side_stream):
                bucket.sync(self._backend, self._dp_group, self._mean_divisor, group_size=self._sync_group_size)
                if self.after_bucket_sync is not None:
                    self.after_bucket_sync(bucket)
                event = self._bucket_events.get(id(bucket))
                if event is None:
                    event = self._bucket_events[id(bucket)] = torch.cuda.Event()
                event.record(self._side_stream)
            self._issued.append(bucket)
            self._side_used = True
        else:
            bucket.sync(self._backend, self._dp_group, self._mean_divisor, group_size=self._sync_group_size)
            if self.after_bucket_sync is not None:
                self.after_bucket_sync(bucket)

    # --------------------------------------------------------------- forward --
    def forward(self, *args: Any, **kwargs: Any) -> Any:
        self._sync_done = False
        return self.module(*args, **kwargs)

    def finish_grad_sync(self, *, join: bool = True, late_buckets: int = 0) -> list[nn.Parameter]:
        """Reduce every bucket not reduced yet; idempotent until the next forward/backward.

        With ``join=False`` the compute stream is NOT made to wait for the last
        ``late_buckets`` reductions issued on the side stream (the buckets that
        only became complete at the very end of the backward pass: the first
        layers, the tied embedding): the parameters of those buckets are
        returned, the caller may work on everything else in the meantime (the
        optimizer update of the other parameters) and must call
        :meth:`join_grad_sync` before touching the returned parameters'
        gradients."""
        if self._sync_done:
            return []
        if self._persistent:
            active = True
        else:
            any_grad = any(p.grad is not None for p in self._param_to_bucket)
            any_activity = any(b.coalesced or b.has_pending_ready for b in self._buckets)
            active = any_grad or any_activity
        late: list[nn.Parameter] = []
        if active:
            for bucket in self._buckets:
                if bucket.coalesced:
                    continue
                if not self._persistent:
                    missing = [p for p in bucket.params if p.grad is None]
                    if missing:
                        names = [self._param_names.get(id(p), "<unknown>") for p in missing]
                        raise RuntimeError(f"finish_grad_sync rank={self._ctx.rank}: missing grads for {names}")
                self._sync_bucket(bucket)
            if self._side_used:
                cur = torch.cuda.current_stream()
                keep = min(late_buckets, len(self._issued)) if not join else 0
                if keep == 0:
                    cur.wait_stream(self._side_stream)
                    self._side_used = False
                else:
                    # the side stream runs the reductions in order: waiting for the last
                    # early one covers all before it
                    early = self._issued[: len(self._issued) - keep]
                    if early:
                        cur.wait_event(self._bucket_events[id(early[-1])])
                    for b in self._issued[len(self._issued) - keep:]:
                        late.extend(b.params)
            for bucket in self._buckets:
                bucket.reset()
            self._write_counts.clear()
            self._issued = []
        self._sync_done = True
        return late

    def join_grad_sync(self) -> None:
        """Make the compute stream wait for reductions left running by
        ``finish_grad_sync(join=False)``."""
        if self._side_used:
            torch.cuda.current_stream().wait_stream(self._side_stream)
            self._side_used = False

    def zero_grad(self, set_to_none: bool = True) -> None:
        """With persistent buffers the gradients are zeroed in place (they stay
        views of the bucket buffers whatever ``set_to_none`` says)."""
        if not self._persistent:
            super().zero_grad(set_to_none=set_to_none)
            return
        if self._overwrite_first and self._zero_plan is None:
            self._learn_zero_plan()
        if self._zero_plan is not None:
            ranges, covered = self._zero_plan
            for i, lo, hi in ranges:
                self._flat_buffers[i][lo:hi].zero_()
            for p in covered:
                p._nmb_overwrite_next = True
        else:
            for flat in self._flat_buffers:
                flat.zero_()
        for b in self._buckets:
            for p, view in zip(b.params, b._views):
                p.grad = view

    def _learn_zero_plan(self) -> None:
        """With ``overwrite_first_grad`` the memset of the gradient buffers is replaced,
        for every parameter whose first gradient write of a step comes from a kernel
        that can store instead of add (weight-gradient GEMMs, bias column sums, norm
        backward), by a flag that makes that first write overwrite.  Which parameters
        qualify is learnt from one traced backward pass between two ``zero_grad``
        calls; the rest (scatter-added embeddings, gradients that arrive through
        autograd) keep being zeroed, as merged ranges of the flat buffers.  Only for
        callers that run exactly one backward pass per ``zero_grad`` with a static
        model (``Trainer``): a parameter that qualified and then receives no gradient
        in some step would keep its previous gradient."""
        from ..ops import functional as F

        if self._grad_trace is None:                      # first call: trace the coming backward pass
            trace = self._grad_trace = {}
            F._GRAD_TRACES.append(trace)
            # a wrapper that is dropped before it finished learning must not stay registered
            weakref.finalize(self, lambda t=trace: F._GRAD_TRACES.__setitem__(
                slice(None), [x for x in F._GRAD_TRACES if x is not t]))
            return
        if not self._grad_trace:                          # no backward pass ran in between: keep tracing
            return
        trace, self._grad_trace = self._grad_trace, None
        F._GRAD_TRACES[:] = [t for t in F._GRAD_TRACES if t is not trace]
        ranges: list[tuple[int, int, int]] = []
        covered: list[nn.Parameter] = []
        for i, b in enumerate(self._buckets):
            offset = 0
            for p in b.params:
                n = p.numel()
                if trace.get(id(p)) == "direct" and not getattr(p, "_nmb_sp_replicated", False):
                    covered.append(p)
                elif ranges and ranges[-1][0] == i and ranges[-1][2] == offset:
                    ranges[-1] = (i, ranges[-1][1], offset + n)
                else:
                    ranges.append((i, offset, offset + n))
                offset += n
        if not covered or len(ranges) > len(self._flat_buffers):
            self._overwrite_first = False                 # would cost more launches than it saves
            return
        self._zero_plan = (ranges, covered)
