"""GEMMs with the tensor/sequence-parallel collective fused into the kernel.

Sequence-parallel Megatron layers pair every GEMM with a collective: all-gather
before a column-parallel GEMM, reduce-scatter after a row-parallel one, and the
mirror images in backward.  The reference issues them as separate blocking NCCL
calls around ``F.linear`` (nano_megatron/parallel/mappings.py:109-163,408-463).
Here each pair is ONE launch of the tcgen05 GEMM (``csrc/gemm_tcgen05.cu``,
``FusedComm``) working on symmetric memory:

* ``allgather_gemm``      -- copy CTAs pull the peers' sequence shards into the
  local full buffer tile by tile while the compute CTAs start on the local
  shard; a tile's TMA loads wait for its ready flag;
* ``gemm_reduce_scatter`` -- a rank computes the other ranks' row blocks first
  and stores each partial tile into the owner's staging slot over NVLink with a
  per-tile flag; its own blocks come last, and their epilogue adds the peers'
  partials (already there), bias and residual -- no separate reduction pass;
* ``gemm_all_reduce``     -- the same with the owner writing the final tile to
  every rank (tensor parallelism without sequence parallelism: the reference's
  ``_ReduceFromTPRegion`` after a row-parallel GEMM and ``_CopyToTPRegion``
  backward after a column-parallel dgrad, nano_megatron/parallel/mappings.py:226-286).

The autograd functions below give the column / row linears (with and without
sequence parallelism) their forward and backward in terms of these launches.
"""
from __future__ import annotations

import ctypes
import os
from typing import Any, Optional

import torch
from torch import Tensor

from . import kernels, native
from .functional import _deliver_grad
from .gemm import (EPI_DGELU, EPI_DSWIGLU, EPI_GELU, EPI_PLAIN, EPI_ROPE, EPI_SWIGLU, RopeSpec, epilogue_extra,
                   gemm_bf16)
from ..utils.tracing import nvtx_range

_MAX = 8
#: CTAs of an all-gather -> GEMM launch that only copy (NMB_AG_COPY_CTAS overrides)
COPY_CTAS = int(os.environ.get("NMB_AG_COPY_CTAS", "16"))
#: switched on by ``enable_symmetric_memory``
ENABLED = False
#: launches of the fused kernels by this process (tests assert on it)
STATS = {"allgather_gemm": 0, "gemm_reduce_scatter": 0, "gemm_all_reduce": 0, "nvlink_bytes": 0}
#: Microbatch slot whose buffers the sequence-parallel call sites use.  A
#: pipeline schedule keeps several microbatches in flight; each one's gathered
#: inputs must survive until its backward pass, so the per-call-site buffers
#: are keyed by (site, slot).
CURRENT_SLOT = 0


class _FusedComm(ctypes.Structure):
    _fields_ = [
        ("ag_src", ctypes.c_void_p * _MAX), ("ag_dst", ctypes.c_void_p), ("ag_ready", ctypes.c_void_p),
        ("ag_copy_ctas", ctypes.c_int), ("rs_mode", ctypes.c_int),
        ("rs_stage", ctypes.c_void_p * _MAX), ("rs_out", ctypes.c_void_p * _MAX),
        ("rs_flags", ctypes.c_void_p * _MAX), ("rs_started", ctypes.c_void_p * _MAX),
        ("rs_last", ctypes.c_void_p * 2),
        ("rs_bias", ctypes.c_void_p), ("rs_residual", ctypes.c_void_p),
        ("pads", ctypes.c_void_p * _MAX), ("sync", ctypes.c_void_p),
        ("channel", ctypes.c_int), ("rank", ctypes.c_int), ("n_ranks", ctypes.c_int),
        ("seq_len", ctypes.c_int), ("shard_len", ctypes.c_int), ("rows_per_rank", ctypes.c_int),
        ("budget", ctypes.c_longlong),
    ]


class TPFused:
    """Per-TP-group state of the fused kernels: staging buffers, flags, counters."""

    def __init__(self, ws: Any) -> None:
        from ..distributed.symm_mem import CHANNEL_TP

        self.ws = ws
        self.channel = CHANNEL_TP
        assert native.lib().nmb_fused_comm_size() == ctypes.sizeof(_FusedComm), "FusedComm layout mismatch"
        #: [0] epoch of the last finished fused launch, [1] CTAs that have left the running one
        self.sync = torch.zeros(2, dtype=torch.int32, device=ws.device)
        self.ready = torch.zeros(4096, dtype=torch.int32, device=ws.device)
        self.max_tiles = int(native.lib().nmb_fused_max_tiles())
        #: per-tile flags written by the peers: [partial stored | final stored][tile][rank]
        #: followed by [rank] "has started the fused launch with this epoch"
        self.flags = ws.alloc_tensor(2 * self.max_tiles * _MAX + _MAX, torch.int32)
        self._flag_ptrs = ws.peers_of(self.flags)
        #: epoch of the last fused launch that used each staging / output buffer
        self.buf_last = torch.zeros(256, dtype=torch.int32, device=ws.device)
        self._buf_index: dict[int, int] = {}
        self._stage: dict[tuple, list[Tensor]] = {}
        self._stage_turn: dict[tuple, int] = {}
        self._gather: dict[tuple, Tensor] = {}

    # -- buffers ---------------------------------------------------------------
    def staging(self, rows: int, cols: int, kind: str = "partial") -> Tensor:
        """Double-buffered symmetric area of ``rows * cols`` bf16 (a rank may run
        one fused op ahead of its peers): ``[n_ranks, rows/n_ranks, cols]``
        partial tiles, or (``kind="out"``) an all-reduced ``[rows, cols]`` result."""
        key = (kind, rows, cols)
        if key not in self._stage:
            self._stage[key] = [self.ws.alloc_tensor(rows * cols, torch.bfloat16) for _ in range(2)]
            self._stage_turn[key] = 0
        turn = self._stage_turn[key]
        self._stage_turn[key] = turn ^ 1
        return self._stage[key][turn]

    def _last_word(self, buf: Tensor) -> int:
        """Address of the device word that records the last launch that used ``buf``."""
        idx = self._buf_index.setdefault(buf.data_ptr(), len(self._buf_index))
        if idx >= self.buf_last.numel():
            raise RuntimeError("too many distinct fused-reduce buffers")
        return self.buf_last.data_ptr() + 4 * idx

    def gather_buffer(self, rows: int, cols: int, *, owner: Any = None) -> Tensor:
        """Symmetric ``[rows, cols]`` buffer for a gathered activation.  With
        ``owner`` the buffer is private to that call site (it is kept for the
        backward pass); otherwise one buffer per shape is shared."""
        if owner is None:
            key = (rows, cols)
        else:
            tag = owner if isinstance(owner, (tuple, str, int)) else id(owner)
            key = (tag, CURRENT_SLOT, rows * cols)
        buf = self._gather.get(key)
        if buf is None:
            buf = self.ws.alloc_tensor(rows * cols, torch.bfloat16).view(rows, cols)
            self._gather[key] = buf
        return buf

    def _base(self, seq_len: int, rows: int) -> _FusedComm:
        ws = self.ws
        fc = _FusedComm()
        for i, p in enumerate(ws.pad.peer_ptrs):
            fc.pads[i] = p
        for i, p in enumerate(self._flag_ptrs):
            fc.rs_flags[i] = p
            fc.rs_started[i] = p + 2 * self.max_tiles * _MAX * 4
        fc.sync = self.sync.data_ptr()
        fc.channel = self.channel
        fc.rank, fc.n_ranks = ws.rank, ws.size
        fc.seq_len, fc.shard_len = seq_len, seq_len // ws.size
        fc.rows_per_rank = rows // ws.size
        fc.budget = ws.budget
        return fc

    def supported(self, rows: int, seq_len: int, n_out: int) -> bool:
        """Whole 128-row tiles per sequence shard, whole 32-column chunks, and the
        tile counts within the flag arrays."""
        t = self.ws.size
        return (seq_len % t == 0 and (seq_len // t) % 128 == 0 and rows % seq_len == 0 and n_out % 32 == 0
                and rows // 128 <= self.ready.numel()
                and (rows // t // 128) * ((n_out + 127) // 128) <= self.max_tiles)

    def all_reduce_supported(self, rows: int, n_out: int) -> bool:
        """The all-reduce treats the rows as one sequence cut into ``t`` blocks."""
        return self.supported(rows, rows, n_out)

    # -- launches ----------------------------------------------------------------
    def _launch(self, a: Tensor, b: Tensor, b_mn: bool, out: Optional[Tensor], m: int, n: int, k: int,
                bias: Optional[Tensor], aux_out: Optional[Tensor], mode: int, fc: _FusedComm,
                rope: Optional[RopeSpec] = None) -> None:
        status = native.status_word(a.device)
        extra = epilogue_extra(rope if mode == EPI_ROPE else None, n // 2 if mode == EPI_SWIGLU else 0)
        rc = native.lib().nmb_gemm_bf16_fused(
            native.ptr(a), ctypes.c_int(a.stride(0)), ctypes.c_int(0), native.ptr(b), ctypes.c_int(b.stride(0)),
            ctypes.c_int(int(b_mn)), native.ptr(out), ctypes.c_int(out.stride(0) if out is not None else n),
            ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k), native.ptr(bias), native.ptr(aux_out),
            ctypes.c_int(mode), ctypes.c_float(1.0), ctypes.byref(fc),
            ctypes.byref(extra) if extra is not None else None, native.ptr(status), native.stream_ptr(a.device))
        native.check_rc(rc, "nmb_gemm_bf16_fused")

    def gemm_reduce_scatter(self, a: Tensor, b: Tensor, seq_len: int, *, b_mn: bool = False,
                            bias: Optional[Tensor] = None, residual: Optional[Tensor] = None) -> Tensor:
        """``reduce_scatter_over_sequence(a @ B^T) + bias + residual`` -> ``[rows/t, n]``.

        ``a`` is ``[rows, k]`` with rows ordered ``[batch][sequence]``; logical B
        is ``[n, k]`` (``b_mn``: stored ``[k, n]``)."""
        m, k = a.shape
        n = b.shape[1] if b_mn else b.shape[0]
        stage = self.staging(m, n)
        out = torch.empty((m // self.ws.size, n), dtype=torch.bfloat16, device=a.device)
        fc = self._base(seq_len, m)
        fc.rs_mode = 1
        fc.rs_last[0] = self._last_word(stage)
        for i, p in enumerate(self.ws.peers_of(stage)):
            fc.rs_stage[i] = p
        fc.rs_out[self.ws.rank] = out.data_ptr()
        fc.rs_bias = bias.data_ptr() if bias is not None else None
        fc.rs_residual = residual.data_ptr() if residual is not None else None
        with nvtx_range("gemm_reduce_scatter"):
            self._launch(a, b, b_mn, None, m, n, k, None, None, EPI_PLAIN, fc)
        STATS["gemm_reduce_scatter"] += 1
        # bytes this rank stores into peers' staging slots (its partial rows they own)
        STATS["nvlink_bytes"] += m * n * 2 * (self.ws.size - 1) // self.ws.size
        return out

    def gemm_all_reduce(self, a: Tensor, b: Tensor, *, b_mn: bool = False, bias: Optional[Tensor] = None,
                        residual: Optional[Tensor] = None) -> Tensor:
        """``sum_over_ranks(a @ B^T) + bias + residual`` -> ``[rows, n]`` on every rank.

        Two-shot inside the GEMM: the rows are cut into one block per rank; the
        owner of a block receives the peers' partial tiles, adds them to its own
        accumulator (+ bias + residual) and writes the final tile into every
        rank's symmetric output; the result is then copied into an ordinary
        tensor so that the caller may keep it for as long as it likes."""
        m, k = a.shape
        n = b.shape[1] if b_mn else b.shape[0]
        stage = self.staging(m, n)
        out_sym = self.staging(m, n, "out")
        fc = self._base(m, m)
        fc.rs_mode = 2
        fc.rs_last[0] = self._last_word(stage)
        fc.rs_last[1] = self._last_word(out_sym)
        for i, p in enumerate(self.ws.peers_of(stage)):
            fc.rs_stage[i] = p
        for i, p in enumerate(self.ws.peers_of(out_sym)):
            fc.rs_out[i] = p
        fc.rs_bias = bias.data_ptr() if bias is not None else None
        fc.rs_residual = residual.data_ptr() if residual is not None else None
        with nvtx_range("gemm_all_reduce"):
            self._launch(a, b, b_mn, None, m, n, k, None, None, EPI_PLAIN, fc)
        STATS["gemm_all_reduce"] += 1
        # partial tiles to the owners plus final tiles to everyone else
        STATS["nvlink_bytes"] += 2 * m * n * 2 * (self.ws.size - 1) // self.ws.size
        return out_sym.view(m, n).clone()

    def allgather_gemm(self, full: Tensor, b: Tensor, seq_len: int, *, b_mn: bool = False,
                       bias: Optional[Tensor] = None, mode: int = EPI_PLAIN,
                       aux_out: Optional[Tensor] = None, rope: Optional[RopeSpec] = None) -> Tensor:
        """``full @ B^T`` where only this rank's sequence shard of the symmetric
        buffer ``full`` is valid on entry; on return ``full`` holds every shard."""
        m, k = full.shape
        n = b.shape[1] if b_mn else b.shape[0]
        out = torch.empty((m, n // 2 if mode == EPI_SWIGLU else n), dtype=torch.bfloat16, device=full.device)
        fc = self._base(seq_len, m)
        fc.ag_copy_ctas = COPY_CTAS
        fc.ag_dst = full.data_ptr()
        fc.ag_ready = self.ready.data_ptr()
        for i, p in enumerate(self.ws.peers_of(full)):
            fc.ag_src[i] = p
        with nvtx_range("allgather_gemm"):
            self._launch(full, b, b_mn, out, m, n, k, bias, aux_out, mode, fc, rope)
        STATS["allgather_gemm"] += 1
        # bytes the copy CTAs pull from the peers' shards
        STATS["nvlink_bytes"] += m * k * 2 * (self.ws.size - 1) // self.ws.size
        return out


def tp_fused_for(group: Any) -> Optional[TPFused]:
    from ..distributed import symmetric

    ws = symmetric.workspace_for(group)
    if ws is None:
        return None
    st = getattr(ws, "_tp_fused", None)
    if st is None:
        st = TPFused(ws)
        ws._tp_fused = st
    return st


def _place_shard(full: Tensor, shard: Tensor, rank: int, seq_len: int, size: int) -> None:
    """Write this rank's ``[B, S/t, K]`` shard into its rows of the ``[B*S, K]`` buffer."""
    b = full.shape[0] // seq_len
    width = seq_len // size
    full.view(b, seq_len, -1)[:, rank * width:(rank + 1) * width].copy_(shard.reshape(b, width, -1))


def _act_mode(act: Optional[str], rope: Optional[RopeSpec]) -> int:
    if act == "swiglu":
        return EPI_SWIGLU
    if act == "gelu":
        return EPI_GELU
    return EPI_ROPE if rope is not None else EPI_PLAIN


class _SPColumnLinearFn(torch.autograd.Function):
    """Sequence-parallel column linear: all-gather -> GEMM (+bias, + activation
    split or rotary epilogue).  With ``act`` it returns ``(pre, act(pre))``."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Optional[Tensor], st: TPFused, seq_len: int, site: Any,
                act: Optional[str], rope: Optional[RopeSpec] = None):
        bsz, width, k = x.shape
        rows = bsz * seq_len
        full = st.gather_buffer(rows, k, owner=site)
        _place_shard(full, x, st.ws.rank, seq_len, st.ws.size)
        n = weight.shape[0]
        pre = torch.empty((rows, n), dtype=torch.bfloat16, device=x.device) if act else None
        y = st.allgather_gemm(full, weight, seq_len, bias=bias, mode=_act_mode(act, rope), aux_out=pre, rope=rope)
        ctx.save_for_backward(full, weight)
        ctx.meta = (st, seq_len, (weight, bias), x.shape)
        if act:
            y = y.view(bsz, seq_len, y.shape[-1])
            ctx.mark_non_differentiable(y)
            ctx.set_materialize_grads(False)
            return pre.view(bsz, seq_len, n), y
        return y.view(bsz, seq_len, n)

    @staticmethod
    def backward(ctx, dy: Optional[Tensor], *_unused):
        full, weight = ctx.saved_tensors
        st, seq_len, (w_param, b_param), in_shape = ctx.meta
        if dy is None:
            return (None,) * 8
        n = weight.shape[0]
        dz = dy.reshape(-1, n)
        if dz.stride(-1) != 1 or dz.stride(0) % 8 != 0:
            dz = dz.contiguous()
        # dgrad partial -> reduce-scatter back to the sequence shard
        dx = st.gemm_reduce_scatter(dz, weight, seq_len, b_mn=True).view(in_shape)
        dw = _deliver_grad(w_param, lambda out, acc: gemm_bf16(dz, full, a_mn=True, b_mn=True, out=out, accumulate=acc))
        db = None
        if b_param is not None:
            db = _deliver_grad(b_param, lambda out, acc: kernels.col_sum(dz, out=out, accumulate=acc))
        return dx, dw, db, None, None, None, None, None


class _SPRowLinearFn(torch.autograd.Function):
    """Sequence-parallel row linear: GEMM -> reduce-scatter (+bias, +residual)."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Optional[Tensor], residual: Optional[Tensor],
                gelu_pre: Optional[Tensor], st: TPFused, seq_len: int, act: str = "gelu"):
        bsz, s, k = x.shape
        x2 = x.reshape(-1, k)
        if x2.stride(-1) != 1 or x2.stride(0) % 8 != 0:
            x2 = x2.contiguous()
        n = weight.shape[0]
        res2 = residual.reshape(-1, n).contiguous() if residual is not None else None
        out = st.gemm_reduce_scatter(x2, weight, seq_len, bias=bias, residual=res2)
        pre2 = gelu_pre.reshape(-1, gelu_pre.shape[-1]) if gelu_pre is not None else None
        ctx.save_for_backward(x2, weight, pre2)
        ctx.meta = (st, seq_len, (weight, bias), x.shape, residual is not None, act,
                    gelu_pre.shape if gelu_pre is not None else None)
        return out.view(bsz, seq_len // st.ws.size, n)

    @staticmethod
    def backward(ctx, dy: Tensor):
        x2, weight, pre2 = ctx.saved_tensors
        st, seq_len, (w_param, b_param), in_shape, has_res, act, pre_shape = ctx.meta
        n = weight.shape[0]
        rows = x2.shape[0]
        # all-gather dY, then dgrad, then the activation's backward on the pre-activation
        dy_full = st.gather_buffer(rows, n)
        _place_shard(dy_full, dy, st.ws.rank, seq_len, st.ws.size)
        if pre2 is not None:
            dact = st.allgather_gemm(dy_full, weight, seq_len, b_mn=True)
            dx = kernels.swiglu_bwd(pre2, dact) if act == "swiglu" else kernels.gelu_bwd(pre2, dact)
        else:
            dx = st.allgather_gemm(dy_full, weight, seq_len, b_mn=True)
        dw = _deliver_grad(w_param, lambda out, acc: gemm_bf16(dy_full, x2, a_mn=True, b_mn=True, out=out, accumulate=acc))
        db = None
        if b_param is not None:
            dyl = dy.reshape(-1, n)
            dyl = dyl if dyl.is_contiguous() else dyl.contiguous()
            db = kernels.col_sum(dyl)  # partial over this rank's tokens; summed over TP by the SP grad hook
        if pre2 is not None:
            return None, dw, db, (dy if has_res else None), dx.view(pre_shape), None, None, None
        return dx.view(in_shape), dw, db, (dy if has_res else None), None, None, None, None


class _TPColumnLinearFn(torch.autograd.Function):
    """Column-parallel linear on a replicated input (tensor parallelism without
    sequence parallelism): a local GEMM forward; the input gradient is a partial
    sum over the ranks' output shards, so the dgrad GEMM carries the all-reduce
    (the reference's ``_CopyToTPRegion`` backward, nano_megatron/parallel/mappings.py:242-257)."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Optional[Tensor], st: TPFused, act: Optional[str],
                rope: Optional[RopeSpec] = None):
        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        if x2.stride(-1) != 1 or x2.stride(0) % 8 != 0:
            x2 = x2.contiguous()
        n = weight.shape[0]
        ctx.save_for_backward(x2, weight)
        ctx.meta = (st, (weight, bias), x.shape)
        out_shape = (*x.shape[:-1], n)
        if act:
            pre = torch.empty((x2.shape[0], n), dtype=torch.bfloat16, device=x.device)
            y = gemm_bf16(x2, weight, bias=bias, mode=_act_mode(act, None), aux_out=pre)
            y = y.view(*x.shape[:-1], y.shape[-1])
            ctx.mark_non_differentiable(y)
            ctx.set_materialize_grads(False)
            return pre.view(out_shape), y
        return gemm_bf16(x2, weight, bias=bias, mode=_act_mode(None, rope), rope=rope).view(out_shape)

    @staticmethod
    def backward(ctx, dy: Optional[Tensor], *_unused):
        x2, weight = ctx.saved_tensors
        st, (w_param, b_param), in_shape = ctx.meta
        if dy is None:
            return None, None, None, None, None, None
        n = weight.shape[0]
        dz = dy.reshape(-1, n)
        if dz.stride(-1) != 1 or dz.stride(0) % 8 != 0:
            dz = dz.contiguous()
        dx = st.gemm_all_reduce(dz, weight, b_mn=True).view(in_shape) if ctx.needs_input_grad[0] else None
        dw = _deliver_grad(w_param, lambda out, acc: gemm_bf16(dz, x2, a_mn=True, b_mn=True, out=out, accumulate=acc))
        db = None
        if b_param is not None:
            db = _deliver_grad(b_param, lambda out, acc: kernels.col_sum(dz, out=out, accumulate=acc))
        return dx, dw, db, None, None, None


class _TPRowLinearFn(torch.autograd.Function):
    """Row-parallel linear without sequence parallelism: GEMM -> all-reduce
    (+ bias + residual) in one launch (the reference's ``_ReduceFromTPRegion``
    forward followed by the bias add, nano_megatron/parallel/mappings.py:274-281,449-463).
    Backward needs no collective: the output gradient is replicated."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Optional[Tensor], residual: Optional[Tensor],
                gelu_pre: Optional[Tensor], st: TPFused, act: str = "gelu"):
        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        if x2.stride(-1) != 1 or x2.stride(0) % 8 != 0:
            x2 = x2.contiguous()
        n = weight.shape[0]
        res2 = residual.reshape(-1, n).contiguous() if residual is not None else None
        out = st.gemm_all_reduce(x2, weight, bias=bias, residual=res2)
        pre2 = gelu_pre.reshape(-1, gelu_pre.shape[-1]) if gelu_pre is not None else None
        ctx.save_for_backward(x2, weight, pre2)
        ctx.meta = ((weight, bias), x.shape, residual is not None, act,
                    gelu_pre.shape if gelu_pre is not None else None)
        return out.view(*x.shape[:-1], n)

    @staticmethod
    def backward(ctx, dy: Tensor):
        x2, weight, pre2 = ctx.saved_tensors
        (w_param, b_param), in_shape, has_res, act, pre_shape = ctx.meta
        n = weight.shape[0]
        dy2 = dy.reshape(-1, n)
        if dy2.stride(-1) != 1 or dy2.stride(0) % 8 != 0:
            dy2 = dy2.contiguous()
        if pre2 is not None:
            dx = gemm_bf16(dy2, weight, b_mn=True, mode=EPI_DSWIGLU if act == "swiglu" else EPI_DGELU,
                           aux_in=pre2).view(pre_shape)
        else:
            dx = gemm_bf16(dy2, weight, b_mn=True).view(in_shape)
        dw = _deliver_grad(w_param, lambda out, acc: gemm_bf16(dy2, x2, a_mn=True, b_mn=True, out=out, accumulate=acc))
        db = None
        if b_param is not None:
            # replicated bias, replicated dy: every rank computes the same sum
            db = _deliver_grad(b_param, lambda out, acc: kernels.col_sum(dy2, out=out, accumulate=acc))
        d_res = dy if has_res else None
        if pre2 is not None:
            return None, dw, db, d_res, dx, None, None
        return dx, dw, db, d_res, None, None, None
