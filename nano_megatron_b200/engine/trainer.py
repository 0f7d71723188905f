"""Training-step engine: one object that owns the model wrapper, the fused
optimizer and (on a GPU) a CUDA graph of the whole step.

The reference has no training-loop layer beyond its single-device
``reference_train_loop`` (nano_megatron/reference/train_step.py:90-120); its
parallel paths are driven by hand-written loops in the benchmark scripts
(scripts/benchmark_dp.py:212-223).  ``Trainer`` is that loop as an API:

    trainer = Trainer(model, ctx, lr=1e-4)
    loss = trainer.step(input_ids)          # zero-grad, fwd, loss, bwd, grad sync, AdamW
    loss = trainer.forward_backward(ids)    # the same without the optimizer (the reference's
                                            # benchmark step, scripts/benchmark_tp.py:182-186)

On CUDA the step (all kernels, the NCCL or peer-memory gradient reductions and
the optimizer) is captured once into a CUDA graph after a few eager warm-up
steps and replayed afterwards, so the host launches one graph per step instead
of ~700 kernels.  Inputs are copied into static device buffers each step.
Gradient buffers are not zeroed (the first gradient write of a step overwrites),
the optimizer update of most parameters overlaps the reduction of the last
gradient buckets, and ``close()`` releases graphs and hooks when a trainer is
discarded.
"""
from __future__ import annotations

from typing import Any, Callable, Optional

import torch
from torch import Tensor, nn

from ..distributed.ddp import DistributedDataParallel
from ..ops import native
from ..utils.tracing import nvtx_range
from ..reference.optimizer import AdamW


class Trainer:
    def __init__(self, model: nn.Module, ctx: Any, *, lr: float = 1e-4, weight_decay: float = 0.01,
                 betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, bucket_cap_mb: float = 25.0,
                 use_cuda_graph: Optional[bool] = None, graph_warmup: int = 3,
                 loss_fn: Optional[Callable[[Tensor, Tensor], Tensor]] = None,
                 overlap_optimizer: Optional[bool] = None) -> None:
        self.model = model
        self.ctx = ctx
        self.graph_error: Optional[str] = None
        # one backward pass per zero_grad and a static model: the first gradient write of a
        # step may overwrite instead of a memset + add (see DistributedDataParallel.zero_grad)
        self.ddp = DistributedDataParallel(model, ctx, bucket_cap_mb=bucket_cap_mb, overwrite_first_grad=True)
        self.optimizer = AdamW(model.named_parameters(), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self._loss_fn = loss_fn or model.shifted_cross_entropy
        #: reductions the optimizer update overlaps with (see ``_step_body``)
        self._late_buckets = 3
        self.device = next(model.parameters()).device
        on_gpu = self.device.type == "cuda"
        # Optional (off by default): update each bucket's parameters as soon as its gradients
        # are final, on a side stream, while backward continues.  It is safe (nothing later in
        # the backward pass reads those weights: a bucket completes after the dgrad and wgrad
        # GEMMs of all its layers, the tied embedding's gradient is the last to complete) but
        # it measured SLOWER: 16.21 ms against 15.98 ms per GPT-345M step on one GPU.  The
        # update's thousands of blocks take SM slots between the one-CTA-per-SM GEMM and
        # attention kernels and delay their CTAs more than the hidden HBM time is worth.
        self._overlap_optimizer = bool(overlap_optimizer) and on_gpu and self.ddp._persistent
        self._opt_stream = torch.cuda.Stream(device=self.device, priority=-1) if on_gpu else None
        self._opt_used = False
        self._bucket_ids: dict[int, set[int]] = {}
        self._want_graph = on_gpu if use_cuda_graph is None else (use_cuda_graph and on_gpu)
        if self._want_graph and not self._collectives_are_graph_safe():
            # Library (NCCL) collectives would land inside the capture; that
            # combination is left eager here.  The peer-memory kernels of this
            # package are plain kernels and capture like any other.
            self._want_graph = False
            self.graph_error = "not captured: the step contains NCCL collectives"
        #: captured step graphs, keyed by "with optimizer update?"
        self._graphs: dict[bool, torch.cuda.CUDAGraph] = {}
        self._tried: set[bool] = set()
        self._pool = None
        self._graph_warmup = graph_warmup
        self._eager_steps = {True: 0, False: 0}
        self._ids: Optional[Tensor] = None
        self._labels: Optional[Tensor] = None
        self._loss_out: Optional[Tensor] = None
        #: number of this library's kernels recorded in the captured graph
        self.kernels_in_graph = 0
        self.kernels_in_graphs: dict[bool, int] = {}

    def _collectives_are_graph_safe(self) -> bool:
        ctx = self.ctx
        if getattr(ctx, "world_size", 1) == 1:
            return True
        if ctx.pipeline_parallel_size > 1:
            return False
        if ctx.tensor_parallel_size > 1:
            # every TP collective (with or without sequence parallelism) on peer-memory kernels
            from ..distributed import symmetric
            from ..ops import fused_tp
            if not (fused_tp.ENABLED and symmetric.workspace_for(ctx.tensor_parallel_group) is not None):
                return False
        if ctx.context_parallel_size > 1:
            from ..distributed import symmetric
            if symmetric.workspace_for(ctx.context_parallel_group) is None:
                return False
        if ctx.data_parallel_size * ctx.context_parallel_size == 1:
            return True                     # no gradient reduction at all
        return all(b.fused_reduce is not None for b in self.ddp._buckets)

    # ------------------------------------------------------------------ step --
    def _update_bucket(self, bucket: Any) -> None:
        """Optimizer update of one gradient bucket (callback of the data-parallel wrapper)."""
        ids = self._bucket_ids.get(id(bucket))
        if ids is None:
            ids = self._bucket_ids[id(bucket)] = {id(p) for p in bucket.params}
        cur = torch.cuda.current_stream(self.device)
        side = self.ddp._side_stream
        if side is not None and cur == side:
            self.optimizer.step(only=ids)          # already ordered after the bucket's reduction
            return
        self._opt_stream.wait_stream(cur)          # the bucket's gradients are final at this point
        with torch.cuda.stream(self._opt_stream):
            self.optimizer.step(only=ids)
        self._opt_used = True

    def _step_body(self, with_optimizer: bool = True) -> Tensor:
        overlap = with_optimizer and self._overlap_optimizer
        self.ddp.after_bucket_sync = self._update_bucket if overlap else None
        with nvtx_range("zero_grad"):
            self.ddp.zero_grad()
        with nvtx_range("forward"):
            logits = self.ddp(self._ids)
            loss = self._loss_fn(logits, self._labels)
        with nvtx_range("backward"):
            loss.backward()
        if overlap:
            with nvtx_range("grad_sync+optimizer"):
                self.ddp.finish_grad_sync()        # what is left: reduce, update; joins the reduction stream
                self.ddp.after_bucket_sync = None
                if self._opt_used:
                    torch.cuda.current_stream(self.device).wait_stream(self._opt_stream)
                    self._opt_used = False
        elif with_optimizer:
            # The buckets that complete last (first layers, tied embedding) are still
            # being reduced when backward ends: update all other parameters meanwhile.
            with nvtx_range("grad_sync"):
                late = self.ddp.finish_grad_sync(join=False, late_buckets=self._late_buckets)
            with nvtx_range("optimizer"):
                if late:
                    ids = {id(p) for p in late}
                    self.optimizer.step(exclude=ids)
                    self.ddp.join_grad_sync()
                    self.optimizer.step(only=ids)
                else:
                    self.ddp.join_grad_sync()
                    self.optimizer.step()
        else:
            with nvtx_range("grad_sync"):
                self.ddp.finish_grad_sync()
        # The loss is handed out in a buffer of its own so that replaying one
        # captured graph never overwrites the value returned by the other.
        self._loss_out.copy_(loss.detach())
        return self._loss_out

    def _load(self, input_ids: Tensor, labels: Optional[Tensor]) -> None:
        if self._ids is None:
            self._ids = torch.empty(input_ids.shape, dtype=torch.long, device=self.device)
            self._labels = torch.empty(input_ids.shape, dtype=torch.long, device=self.device)
            self._loss_out = torch.zeros((), dtype=torch.float32, device=self.device)
        self._ids.copy_(input_ids, non_blocking=True)
        self._labels.copy_(input_ids if labels is None else labels, non_blocking=True)

    def step(self, input_ids: Tensor, labels: Optional[Tensor] = None) -> Tensor:
        """One optimisation step; returns the (device) scalar loss."""
        return self._run(input_ids, labels, True)

    def forward_backward(self, input_ids: Tensor, labels: Optional[Tensor] = None) -> Tensor:
        """Zero-grad, forward, loss, backward and gradient synchronisation, no
        parameter update: gradients are left in ``.grad`` for the caller."""
        return self._run(input_ids, labels, False)

    def _run(self, input_ids: Tensor, labels: Optional[Tensor], with_optimizer: bool) -> Tensor:
        self._load(input_ids, labels)
        graph = self._graphs.get(with_optimizer)
        if graph is None and self._want_graph and with_optimizer not in self._tried \
                and self._eager_steps[with_optimizer] >= self._graph_warmup:
            graph = self._capture(with_optimizer)
        if graph is not None:
            if with_optimizer:
                self.optimizer.sync_hyper()      # a changed lr reaches the device outside the graph
            graph.replay()
            return self._loss_out
        self._eager_steps[with_optimizer] += 1
        return self._step_body(with_optimizer)

    def _capture(self, with_optimizer: bool) -> Optional[torch.cuda.CUDAGraph]:
        """Capture the whole step.  A failure leaves that kind of step in eager
        mode (``graph_error`` says why)."""
        self._tried.add(with_optimizer)
        torch.cuda.synchronize(self.device)
        try:
            graph = torch.cuda.CUDAGraph()
            before = native.launches
            kwargs = {} if self._pool is None else {"pool": self._pool}
            with torch.cuda.graph(graph, capture_error_mode="thread_local", **kwargs):
                self._step_body(with_optimizer)
            if self._pool is None:
                self._pool = graph.pool()
            if with_optimizer or not self.kernels_in_graph:
                self.kernels_in_graph = native.launches - before
            self.kernels_in_graphs[with_optimizer] = native.launches - before
            self._graphs[with_optimizer] = graph
            return graph
        except Exception as exc:  # pragma: no cover - depends on the device
            self.graph_error = f"{type(exc).__name__}: {exc}"
            torch.cuda.synchronize(self.device)
            return None

    def graph_settled(self, with_optimizer: bool) -> bool:
        """True once that kind of step will not change mode any more: it is captured, its
        capture was tried and failed, or graphs are not wanted.  A benchmark calls the step
        until this holds so that no timed region contains a capture."""
        return (not self._want_graph) or with_optimizer in self._graphs or with_optimizer in self._tried

    def reset_graphs(self) -> None:
        """Drop the captured graphs (they are re-captured after the usual eager
        warm-up).  Needed after anything that moves a tensor the graphs address:
        re-created optimizer state, re-bound gradient buffers."""
        self._graphs.clear()
        self._tried.clear()
        self._eager_steps = {True: 0, False: 0}

    @property
    def graphed(self) -> bool:
        return bool(self._graphs)

    def close(self) -> None:
        """Drop the captured graphs and detach the data-parallel wrapper from the model (its
        hooks keep model and gradient buffers alive otherwise).  Call it when the trainer is
        discarded and the process goes on, with no step in flight."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self._graphs.clear()
        self._tried.clear()
        self._pool = None
        self.ddp.close()

    def check(self) -> None:
        """Raise if any kernel reported a device-side failure (host sync)."""
        if self.device.type == "cuda":
            native.check_status(self.device)
