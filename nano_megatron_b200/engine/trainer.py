"""Training-step engine: one object that owns the model wrapper, the fused
optimizer and (on a GPU) a CUDA graph of the whole step.

The reference has no training-loop layer beyond its single-device
``reference_train_loop`` (nano_megatron/reference/train_step.py:90-120); its
parallel paths are driven by hand-written loops in the benchmark scripts
(scripts/benchmark_dp.py:212-223).  ``Trainer`` is that loop as an API:

    trainer = Trainer(model, ctx, lr=1e-4)
    loss = trainer.step(input_ids)          # zero-grad, fwd, loss, bwd, grad sync, AdamW

On CUDA the step (all kernels, the NCCL or peer-memory gradient reductions and
the optimizer) is captured once into a CUDA graph after a few eager warm-up
steps and replayed afterwards, so the host launches one graph per step instead
of ~1500 kernels.  Inputs are copied into static device buffers each step.
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
                 loss_fn: Optional[Callable[[Tensor, Tensor], Tensor]] = None) -> None:
        self.model = model
        self.ctx = ctx
        self.graph_error: Optional[str] = None
        self.ddp = DistributedDataParallel(model, ctx, bucket_cap_mb=bucket_cap_mb)
        self.optimizer = AdamW(model.named_parameters(), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self._loss_fn = loss_fn or model.shifted_cross_entropy
        self.device = next(model.parameters()).device
        on_gpu = self.device.type == "cuda"
        self._want_graph = on_gpu if use_cuda_graph is None else (use_cuda_graph and on_gpu)
        if self._want_graph and not self._collectives_are_graph_safe():
            # Library (NCCL) collectives would land inside the capture; that
            # combination is left eager here.  The peer-memory kernels of this
            # package are plain kernels and capture like any other.
            self._want_graph = False
            self.graph_error = "not captured: the step contains NCCL collectives"
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._graph_warmup = graph_warmup
        self._eager_steps = 0
        self._ids: Optional[Tensor] = None
        self._labels: Optional[Tensor] = None
        self._loss: Optional[Tensor] = None
        #: number of this library's kernels recorded in the captured graph
        self.kernels_in_graph = 0

    def _collectives_are_graph_safe(self) -> bool:
        ctx = self.ctx
        if getattr(ctx, "world_size", 1) == 1:
            return True
        if ctx.pipeline_parallel_size > 1:
            return False
        if ctx.tensor_parallel_size > 1:
            # sequence-parallel TP with every collective on peer-memory kernels
            from ..distributed import symmetric
            from ..ops import fused_tp
            if not (ctx.sequence_parallel and fused_tp.ENABLED
                    and symmetric.workspace_for(ctx.tensor_parallel_group) is not None):
                return False
        if ctx.context_parallel_size > 1:
            from ..distributed import symmetric
            if symmetric.workspace_for(ctx.context_parallel_group) is None:
                return False
        if ctx.data_parallel_size * ctx.context_parallel_size == 1:
            return True                     # no gradient reduction at all
        return all(b.fused_reduce is not None for b in self.ddp._buckets)

    # ------------------------------------------------------------------ step --
    def _step_body(self) -> Tensor:
        with nvtx_range("zero_grad"):
            self.ddp.zero_grad()
        with nvtx_range("forward"):
            logits = self.ddp(self._ids)
            loss = self._loss_fn(logits, self._labels)
        with nvtx_range("backward"):
            loss.backward()
        with nvtx_range("grad_sync"):
            self.ddp.finish_grad_sync()
        with nvtx_range("optimizer"):
            self.optimizer.step()
        return loss.detach()

    def _load(self, input_ids: Tensor, labels: Optional[Tensor]) -> None:
        if self._ids is None:
            self._ids = torch.empty(input_ids.shape, dtype=torch.long, device=self.device)
            self._labels = torch.empty(input_ids.shape, dtype=torch.long, device=self.device)
        self._ids.copy_(input_ids, non_blocking=True)
        self._labels.copy_(input_ids if labels is None else labels, non_blocking=True)

    def step(self, input_ids: Tensor, labels: Optional[Tensor] = None) -> Tensor:
        """One optimisation step; returns the (device) scalar loss."""
        self._load(input_ids, labels)
        if self._graph is not None:
            self._graph.replay()
            return self._loss
        if self._want_graph and self._eager_steps >= self._graph_warmup:
            self._capture()
            if self._graph is not None:
                self._graph.replay()
                return self._loss
        self._eager_steps += 1
        return self._step_body()

    def _capture(self) -> None:
        """Capture the whole step.  A failure leaves the trainer in eager mode
        (``graph_error`` says why)."""
        self._want_graph = False
        torch.cuda.synchronize(self.device)
        try:
            graph = torch.cuda.CUDAGraph()
            before = native.launches
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self._loss = self._step_body()
            self.kernels_in_graph = native.launches - before
            self._graph = graph
        except Exception as exc:  # pragma: no cover - depends on the device
            self.graph_error = f"{type(exc).__name__}: {exc}"
            self._graph = None
            torch.cuda.synchronize(self.device)

    @property
    def graphed(self) -> bool:
        return self._graph is not None

    def check(self) -> None:
        """Raise if any kernel reported a device-side failure (host sync)."""
        if self.device.type == "cuda":
            native.check_status(self.device)
