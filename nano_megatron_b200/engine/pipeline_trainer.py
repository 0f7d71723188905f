"""Training step for a pipeline stage: non-interleaved 1F1B with the stage's
forward and backward of every microbatch slot captured in CUDA graphs.

The reference drives a pipeline stage with ``forward_backward_1f1b``
(nano_megatron/schedules/one_f_one_b.py:41-322): eager autograd per
microbatch, blocking NCCL send / recv on the compute stream, one gradient
flush at the end.  A stage of a 24-layer model launches ~700 kernels per
microbatch forward + backward, so with 2048-token microbatches the step is
bound by the host.  ``PipelineTrainer`` keeps the schedule (same warm-up count,
same exchange order with the neighbours, loss scaled by ``1/M``, gradients
accumulated over the microbatches and synchronised once) and changes how it is
executed:

* a stage holds at most ``warm-up + 1`` microbatches in flight; each such
  *slot* gets static input / output / gradient buffers and two CUDA graphs
  (forward, backward) with a memory pool of its own, so the activations a
  slot saves for its backward pass are never touched by another slot;
* activations and gradients travel by NCCL point-to-point **outside** the
  graphs, on a communication stream, straight into / out of the slots' static
  buffers (no per-call allocation); CUDA events order them against the
  graph launches, so a send never stalls the compute stream and the next
  receive is already posted while the stage computes;
* the tensor-parallel collectives inside the stage are the peer-memory kernels
  of this package (plain kernels, capturable); if any collective of the stage
  would go through the library (NCCL) the trainer stays eager and says why in
  ``graph_error``.

``step`` = zero-grad, 1F1B forward / backward over the microbatches, gradient
synchronisation over the DP group, AdamW.  ``forward_backward`` stops before
the optimizer.  The last stage returns the loss (sum of the microbatch losses,
each scaled by ``1/M``), the other stages ``None``.
"""
from __future__ import annotations

from contextlib import nullcontext
from typing import Any, Optional

import torch
from torch import Tensor, nn

from ..distributed.ddp import DistributedDataParallel
from ..ops import native
from ..parallel.context import (
    is_pipeline_first_stage,
    is_pipeline_last_stage,
    pipeline_next_rank,
    pipeline_prev_rank,
)
from ..reference.optimizer import AdamW
from ..schedules.one_f_one_b import forward_backward_1f1b, warmup_microbatches


class _Slot:
    """Static buffers and graphs of one in-flight microbatch."""

    def __init__(self) -> None:
        self.x: Optional[Tensor] = None          # ids (first stage) or received activation
        self.labels: Optional[Tensor] = None     # last stage
        self.positions: Optional[Tensor] = None
        self.out: Optional[Tensor] = None        # activation to send on, or the scaled loss
        self.grad_out: Optional[Tensor] = None   # received gradient of `out`
        self.grad_in: Optional[Tensor] = None    # gradient to send back
        self.fwd: Optional[torch.cuda.CUDAGraph] = None
        self.bwd: Optional[torch.cuda.CUDAGraph] = None
        self.ev_in = torch.cuda.Event()          # input received
        self.ev_fwd = torch.cuda.Event()         # forward replay finished
        self.ev_gout = torch.cuda.Event()        # gradient received
        self.ev_bwd = torch.cuda.Event()         # backward replay finished
        self.ev_sent_f = torch.cuda.Event()      # activation sent (out may be overwritten)
        self.ev_sent_b = torch.cuda.Event()      # gradient sent (grad_in may be overwritten)
        self.sent_f = self.sent_b = False


class PipelineTrainer:
    def __init__(self, stage: nn.Module, ctx: Any, *, num_microbatches: int, lr: float = 1e-4,
                 weight_decay: float = 0.01, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 bucket_cap_mb: float = 25.0, use_cuda_graph: Optional[bool] = None, graph_warmup: int = 2) -> None:
        if num_microbatches < 1:
            raise ValueError(f"num_microbatches must be >= 1, got {num_microbatches}")
        self.stage, self.ctx, self.m = stage, ctx, num_microbatches
        self.ddp = DistributedDataParallel(stage, ctx, bucket_cap_mb=bucket_cap_mb)
        self.optimizer = AdamW(stage.named_parameters(), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self.device = next(stage.parameters()).device
        self.dtype = next(stage.parameters()).dtype
        self.first, self.last = is_pipeline_first_stage(ctx), is_pipeline_last_stage(ctx)
        self.prev, self.next = pipeline_prev_rank(ctx), pipeline_next_rank(ctx)
        self.n_warm = warmup_microbatches(ctx.pipeline_parallel_size, ctx.pipeline_parallel_rank, num_microbatches)
        self.graph_error: Optional[str] = None
        on_gpu = self.device.type == "cuda"
        self._want_graph = on_gpu if use_cuda_graph is None else (use_cuda_graph and on_gpu)
        if self._want_graph and not self._stage_collectives_capturable():
            self._want_graph = False
            self.graph_error = "not captured: the stage contains NCCL collectives"
        self._graph_warmup = graph_warmup
        self._eager_steps = 0
        self._slots: list[_Slot] = []
        self._shape: Optional[tuple[int, int]] = None
        self._loss_acc: Optional[Tensor] = None
        self._comm = torch.cuda.Stream(device=self.device) if on_gpu else None
        self.kernels_in_graph = 0

    # ------------------------------------------------------------- predicates --
    def _stage_collectives_capturable(self) -> bool:
        ctx = self.ctx
        if ctx.tensor_parallel_size > 1:
            from ..distributed import symmetric
            from ..ops import fused_tp
            if not fused_tp.ENABLED or symmetric.workspace_for(ctx.tensor_parallel_group) is None:
                return False
        return True

    def _parameters_write_directly(self) -> bool:
        """Every parameter's gradient is accumulated into its bucket buffer by the
        backward kernels themselves (``main_grad``).  Parameters whose gradient
        comes back through autograd (replicated parameters under sequence
        parallelism, whose hook reduces them over the TP group) need the eager
        schedule: the graphed backward of a later stage asks autograd only for the
        gradient of the stage input."""
        return all(getattr(p, "main_grad", None) is not None and not getattr(p, "_nmb_sp_replicated", False)
                   for p in self.stage.parameters() if p.requires_grad)

    @property
    def graphed(self) -> bool:
        return bool(self._slots)

    def close(self) -> None:
        """Drop the captured graphs and detach the data-parallel wrapper from the stage (see
        ``Trainer.close``)."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self._slots = []
        self.ddp.close()

    def check(self) -> None:
        if self.device.type == "cuda":
            native.check_status(self.device)

    # ------------------------------------------------------------------ steps --
    def step(self, input_ids: Tensor, labels: Optional[Tensor] = None) -> Optional[Tensor]:
        loss = self.forward_backward(input_ids, labels)
        self.optimizer.step()
        return loss

    def forward_backward(self, input_ids: Tensor, labels: Optional[Tensor] = None) -> Optional[Tensor]:
        if input_ids.device != self.device:
            input_ids = input_ids.to(self.device, non_blocking=True)
        labels = input_ids if labels is None else labels.to(self.device, non_blocking=True)
        if input_ids.dim() != 2 or input_ids.shape[0] % self.m != 0:
            raise ValueError(f"input_ids must be [B, S] with B divisible by {self.m} microbatches, "
                             f"got {tuple(input_ids.shape)}")
        self.ddp.zero_grad()
        if self._want_graph and not self._slots and self._eager_steps >= self._graph_warmup:
            if not self._parameters_write_directly():
                self._want_graph = False
                self.graph_error = "not captured: some parameter gradients are delivered through autograd"
        if self._want_graph and not self._slots and self._eager_steps >= self._graph_warmup:
            self._capture(input_ids.shape[0] // self.m, input_ids.shape[1])
        if self._slots and self._shape == (input_ids.shape[0] // self.m, input_ids.shape[1]):
            return self._run_graphed(input_ids, labels)
        self._eager_steps += 1
        return forward_backward_1f1b(stage=self.stage, ctx=self.ctx, input_ids=input_ids, labels=labels,
                                     num_microbatches=self.m, ddp=self.ddp)

    # ---------------------------------------------------------------- capture --
    def _capture(self, mb: int, seq: int) -> None:
        """Capture forward and backward of every slot.  Nothing executes during a
        capture, so no rank waits for another here; all ranks of the stage's
        tensor-parallel group record the same kernels in the same order."""
        self._want_graph = False
        where = "set-up"
        stage = self.stage
        n_slots = min(self.n_warm + 1, self.m)
        act_shape = stage.activation_shape(mb, seq)
        slots: list[_Slot] = []
        torch.cuda.synchronize(self.device)
        self._loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        try:
            from ..ops import fused_tp
            before = native.launches
            for s in range(n_slots):
                fused_tp.CURRENT_SLOT = s
                slot = _Slot()
                if self.first:
                    slot.x = torch.zeros((mb, seq), dtype=torch.long, device=self.device)
                else:
                    slot.x = torch.zeros(act_shape, dtype=self.dtype, device=self.device).requires_grad_(True)
                slot.positions = torch.arange(seq, device=self.device).unsqueeze(0).expand(mb, -1).contiguous()
                if self.last:
                    slot.labels = torch.zeros((mb, seq), dtype=torch.long, device=self.device)
                else:
                    slot.grad_out = torch.zeros(act_shape, dtype=self.dtype, device=self.device)
                slot.fwd, slot.bwd = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
                where = f"forward of slot {s}"
                with torch.cuda.graph(slot.fwd, capture_error_mode="thread_local"):
                    out = stage(slot.x, positions=slot.positions)
                    if self.last:
                        out = stage.shifted_cross_entropy(out, slot.labels) / self.m
                        self._loss_acc.add_(out.detach().float())
                    slot.out = out
                pool = slot.fwd.pool()
                where = f"backward of slot {s}"
                with torch.cuda.graph(slot.bwd, pool=pool, capture_error_mode="thread_local"):
                    with self.ddp.no_sync():
                        if self.first:
                            # no differentiable input: parameters only (their gradients are
                            # written into the bucket buffers by the backward kernels)
                            if self.last:
                                slot.out.backward(retain_graph=True)
                            else:
                                torch.autograd.backward(slot.out, grad_tensors=slot.grad_out, retain_graph=True)
                        else:
                            # The input gradient is asked for explicitly, so that no
                            # gradient-accumulation node of a leaf runs inside the capture;
                            # the parameter gradients are side effects of the same backward
                            # functions (checked in _parameters_write_directly).
                            (slot.grad_in,) = torch.autograd.grad(
                                [slot.out], [slot.x], grad_outputs=None if self.last else [slot.grad_out],
                                retain_graph=True)
                slots.append(slot)
            self.kernels_in_graph = (native.launches - before) * self.m // n_slots
            self._slots, self._shape = slots, (mb, seq)
        except Exception as exc:  # pragma: no cover - depends on the device
            import traceback
            frames = traceback.extract_tb(exc.__traceback__)
            trail = " <- ".join(f"{f.name}:{f.lineno}" for f in frames[-4:])
            self.graph_error = f"capture of the {where} failed: {type(exc).__name__}: {str(exc)[:300]} [{trail}]"
            self._slots = []
            torch.cuda.synchronize(self.device)
        finally:
            from ..ops import fused_tp
            fused_tp.CURRENT_SLOT = 0
        # capture ran no kernel: the gradient buffers are still clean for this step

    # ----------------------------------------------------------------- replay --
    def _send(self, tensor: Tensor, dst: int, after: torch.cuda.Event, done: torch.cuda.Event) -> None:
        comm = self._comm
        comm.wait_event(after)
        with torch.cuda.stream(comm):
            self.ctx.backend.send(tensor, dst=dst, group=self.ctx.pipeline_parallel_group)
            done.record(comm)

    def _recv(self, tensor: Tensor, src: int, after: Optional[torch.cuda.Event], done: torch.cuda.Event) -> None:
        comm = self._comm
        if after is not None:
            comm.wait_event(after)
        with torch.cuda.stream(comm):
            self.ctx.backend.recv(tensor, src=src, group=self.ctx.pipeline_parallel_group)
            done.record(comm)

    def _run_graphed(self, input_ids: Tensor, labels: Tensor) -> Optional[Tensor]:
        m, mb = self.m, self._shape[0]
        cur = torch.cuda.current_stream(self.device)
        n_slots = len(self._slots)
        self._loss_acc.zero_()
        for slot in self._slots:
            slot.sent_f = slot.sent_b = False
        used = [False] * n_slots

        def fetch(i: int) -> None:
            """Microbatch i's stage input into its slot (the slot's previous
            backward, the last reader of the buffer, has been launched)."""
            slot = self._slots[i % n_slots]
            if self.first:
                slot.x.copy_(input_ids[i * mb:(i + 1) * mb], non_blocking=True)
            else:
                with torch.no_grad():
                    self._recv(slot.x, self.prev, slot.ev_bwd if used[i % n_slots] else None, slot.ev_in)
            if self.last:
                slot.labels.copy_(labels[i * mb:(i + 1) * mb], non_blocking=True)

        def forward(i: int) -> None:
            slot = self._slots[i % n_slots]
            if not self.first:
                cur.wait_event(slot.ev_in)
            if slot.sent_f:
                cur.wait_event(slot.ev_sent_f)     # the previous activation has left the buffer
            slot.fwd.replay()
            slot.ev_fwd.record(cur)
            used[i % n_slots] = True

        def send_forward(i: int) -> None:
            slot = self._slots[i % n_slots]
            if not self.last:
                self._send(slot.out, self.next, slot.ev_fwd, slot.ev_sent_f)
                slot.sent_f = True

        def recv_backward(i: int) -> None:
            slot = self._slots[i % n_slots]
            if not self.last:
                # the previous gradient in this buffer was consumed by the slot's last backward
                self._recv(slot.grad_out, self.next, slot.ev_bwd if slot.sent_b or used[i % n_slots] else None,
                           slot.ev_gout)

        def backward(i: int) -> None:
            slot = self._slots[i % n_slots]
            if not self.last:
                cur.wait_event(slot.ev_gout)
            if slot.sent_b:
                cur.wait_event(slot.ev_sent_b)     # the previous input gradient has left the buffer
            slot.bwd.replay()
            slot.ev_bwd.record(cur)
            if not self.first:
                self._send(slot.grad_in, self.prev, slot.ev_bwd, slot.ev_sent_b)
                slot.sent_b = True

        n_warm, n_steady = self.n_warm, m - self.n_warm
        for i in range(n_warm):
            fetch(i)
            forward(i)
            send_forward(i)
        if n_steady > 0:
            fetch(n_warm)
        for k in range(n_steady):
            i = n_warm + k
            forward(i)
            recv_backward(i - n_warm)
            send_forward(i)
            backward(i - n_warm)
            if k + 1 < n_steady:
                fetch(i + 1)
        for i in range(m - n_warm, m):
            recv_backward(i)
            backward(i)
        # nothing of this step is still in flight on the communication stream
        cur.wait_stream(self._comm)
        self.ddp._sync_done = False
        self.ddp.finish_grad_sync()
        return self._loss_acc if self.last else None
