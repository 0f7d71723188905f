"""Thin ctypes wrappers around the non-GEMM kernels (norm, cross entropy,
embedding, activations, rotary, AdamW).  Each function launches on the current
stream and returns torch tensors; shapes are validated here so the C side can
stay small."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import native

c_int, c_ll, c_float = ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _bf16(t: torch.Tensor) -> torch.Tensor:
    assert t.is_cuda and t.dtype == torch.bfloat16, "bf16 CUDA tensor expected"
    return t if t.is_contiguous() else t.contiguous()


_scratch: dict[tuple[int, int], torch.Tensor] = {}


def _col_scratch(device: torch.device, h: int) -> torch.Tensor:
    key = (device.index or 0, h)
    buf = _scratch.get(key)
    if buf is None:
        buf = torch.empty(2 * 64 * h, dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


# ------------------------------------------------------------------- norm --
def norm_fwd(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float, rms: bool):
    x = _bf16(x)
    h = x.shape[-1]
    rows = x.numel() // h
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = native.lib().nmb_norm_fwd(native.ptr(x), native.ptr(_bf16(w)), native.ptr(None if b is None else _bf16(b)),
                                   native.ptr(y), native.ptr(mean), native.ptr(rstd), c_int(rows), c_int(h),
                                   c_float(eps), c_int(int(rms)), native.stream_ptr(x.device))
    native.check_rc(rc, "nmb_norm_fwd")
    return y, mean, rstd


_norm_partial: dict[tuple[int, int], torch.Tensor] = {}


def norm_bwd(dy, x, w, mean, rstd, rms: bool, dx_add: Optional[torch.Tensor] = None, want_bias: bool = True,
             grad_out: Optional[tuple] = None, accumulate: bool = True):
    """``(dx, dgamma, dbeta)``.  ``dx_add`` is added to dx (the gradient of a
    residual branch that bypassed the norm).  ``grad_out = (dgamma_buf,
    dbeta_buf)`` makes the kernels write the parameter gradients to those bf16
    buffers (added to their contents, or stored with ``accumulate=False``); the
    returned dgamma / dbeta are then None."""
    dy, x = _bf16(dy), _bf16(x)
    h = x.shape[-1]
    rows = x.numel() // h
    dx = torch.empty_like(x)
    lib = native.lib()
    if dx_add is not None:
        dx_add = _bf16(dx_add)
    acc = grad_out is not None
    add = acc and accumulate
    if h % 256 == 0 and h <= 1024:
        # one pass over dy and x: dx plus the column sums for dgamma / dbeta
        key = (x.device.index or 0, h)
        partial = _norm_partial.get(key)
        if partial is None:
            partial = torch.empty(lib.nmb_norm_bwd_fused_blocks() * 2 * h, dtype=torch.float32, device=x.device)
            _norm_partial[key] = partial
        if acc:
            dw, db = grad_out
        else:
            dw = torch.empty(h, dtype=torch.bfloat16, device=x.device)
            db = torch.empty(h, dtype=torch.bfloat16, device=x.device) if want_bias else None
        rc = lib.nmb_norm_bwd_fused(native.ptr(dy), native.ptr(x), native.ptr(_bf16(w)), native.ptr(mean),
                                    native.ptr(rstd), native.ptr(dx_add), native.ptr(dx), native.ptr(dw),
                                    native.ptr(db), native.ptr(partial), c_int(rows), c_int(h), c_int(int(rms)),
                                    c_int(int(add)), native.stream_ptr(x.device))
        if rc == 0:
            native.launches += 2
            return (dx, None, None) if acc else (dx, dw, db)
        if rc != -1:
            native.check_rc(rc, "nmb_norm_bwd_fused")
    rc = lib.nmb_norm_bwd_dx(native.ptr(dy), native.ptr(x), native.ptr(_bf16(w)), native.ptr(mean), native.ptr(rstd),
                             native.ptr(None if dx_add is None else _bf16(dx_add)), native.ptr(dx), c_int(rows),
                             c_int(h), c_int(int(rms)), native.stream_ptr(x.device))
    native.check_rc(rc, "nmb_norm_bwd_dx")
    if acc:
        dw, db = grad_out
    else:
        dw = torch.empty(h, dtype=torch.bfloat16, device=x.device)
        db = torch.empty(h, dtype=torch.bfloat16, device=x.device) if want_bias else None
    rc = lib.nmb_col_reduce(native.ptr(dy), c_int(h), native.ptr(x), native.ptr(mean), native.ptr(rstd),
                            native.ptr(_col_scratch(x.device, h)), native.ptr(dw), native.ptr(db), c_int(rows),
                            c_int(h), c_int(1), c_int(int(rms)), c_int(int(add)), native.stream_ptr(x.device))
    native.check_rc(rc, "nmb_col_reduce")
    return (dx, None, None) if acc else (dx, dw, db)


def col_sum(dy: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """Sum of a 2-D bf16 tensor over its rows (bias gradient)."""
    assert dy.dim() == 2 and dy.stride(1) == 1
    rows, h = dy.shape
    if out is None:
        out = torch.empty(h, dtype=torch.bfloat16, device=dy.device)
    rc = native.lib().nmb_col_reduce(native.ptr(dy), c_int(dy.stride(0)), native.ptr(None), native.ptr(None),
                                     native.ptr(None), native.ptr(_col_scratch(dy.device, h)), native.ptr(out),
                                     native.ptr(None), c_int(rows), c_int(h), c_int(0), c_int(0),
                                     c_int(int(accumulate)), native.stream_ptr(dy.device))
    native.check_rc(rc, "nmb_col_reduce")
    return out


# ---------------------------------------------------------- cross entropy --
def ce_stats(logits: torch.Tensor, target: torch.Tensor, vocab_start: int) -> torch.Tensor:
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype == torch.bfloat16
    rows, vloc = logits.shape
    stats = torch.empty((rows, 3), dtype=torch.float32, device=logits.device)
    rc = native.lib().nmb_ce_stats(native.ptr(logits), c_ll(logits.stride(0)), native.ptr(target), c_int(vocab_start),
                                   c_int(vloc), native.ptr(stats), c_int(rows), native.stream_ptr(logits.device))
    native.check_rc(rc, "nmb_ce_stats")
    return stats


def ce_combine(all_stats: torch.Tensor, target: torch.Tensor, ignore_index: int, want_rows: bool = False):
    """all_stats: [ranks, rows, 3].  Returns (lse[rows], accum[2] = {loss sum, valid count}, loss_rows|None)."""
    n_ranks, rows, _ = all_stats.shape
    lse = torch.empty(rows, dtype=torch.float32, device=all_stats.device)
    accum = torch.zeros(2, dtype=torch.float32, device=all_stats.device)
    loss_rows = torch.empty(rows, dtype=torch.float32, device=all_stats.device) if want_rows else None
    rc = native.lib().nmb_ce_combine(native.ptr(all_stats), c_int(n_ranks), native.ptr(target), c_int(ignore_index),
                                     native.ptr(lse), native.ptr(loss_rows), native.ptr(accum), c_int(rows),
                                     native.stream_ptr(all_stats.device))
    native.check_rc(rc, "nmb_ce_combine")
    return lse, accum, loss_rows


class _CeComm(ctypes.Structure):
    _fields_ = [("gathered", (ctypes.c_void_p * 8) * 2), ("flags", ctypes.c_void_p * 8), ("sync", ctypes.c_void_p),
                ("rank", c_int), ("n_ranks", c_int), ("budget", c_ll)]


class CeExchange:
    """Buffers of the one-launch cross-entropy forward for a given row count:
    two gather buffers of (max, sum-exp, target logit) triples per rank and row,
    the peers' "all rows stored" flags and the device-side epoch.  With a
    symmetric workspace ``ws`` the buffers are peer-addressable (tensor
    parallelism); without one they are plain local tensors (single rank)."""

    def __init__(self, rows: int, device: torch.device, ws=None) -> None:
        assert native.lib().nmb_ce_comm_size() == ctypes.sizeof(_CeComm), "CeComm layout mismatch"
        self.rows, self.ws = rows, ws
        n = ws.size if ws is not None else 1
        self.sync = torch.zeros(2, dtype=torch.int32, device=device)
        self.comm = _CeComm()
        self._keep = []
        if ws is None:
            for parity in range(2):
                buf = torch.empty(rows * 4, dtype=torch.float32, device=device)
                self._keep.append(buf)
                self.comm.gathered[parity][0] = buf.data_ptr()
            self.comm.rank, self.comm.n_ranks, self.comm.budget = 0, 1, 0
        else:
            flags = ws.alloc_tensor(8, torch.int32)
            self._keep.append(flags)
            for i, p in enumerate(ws.peers_of(flags)):
                self.comm.flags[i] = p
            for parity in range(2):
                buf = ws.alloc_tensor(n * rows * 4, torch.float32)
                self._keep.append(buf)
                for i, p in enumerate(ws.peers_of(buf)):
                    self.comm.gathered[parity][i] = p
            self.comm.rank, self.comm.n_ranks, self.comm.budget = ws.rank, n, ws.budget
        self.comm.sync = self.sync.data_ptr()


def ce_forward_fused(logits: torch.Tensor, target: torch.Tensor, vocab_start: int, ignore_index: int,
                     ex: CeExchange):
    """One launch: per-row statistics, cross-rank exchange, combine.  Returns
    ``(lse[rows], accum[2] = {loss sum, valid count})``."""
    assert logits.dim() == 2 and logits.stride(1) == 1 and logits.dtype == torch.bfloat16
    rows, vloc = logits.shape
    assert rows == ex.rows
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    accum = torch.empty(2, dtype=torch.float32, device=logits.device)
    rc = native.lib().nmb_ce_forward_fused(
        native.ptr(logits), c_ll(logits.stride(0)), native.ptr(target), c_int(vocab_start), c_int(vloc),
        c_int(ignore_index), ctypes.byref(ex.comm), native.ptr(lse), native.ptr(accum), c_int(rows),
        native.ptr(native.status_word(logits.device)), native.stream_ptr(logits.device))
    native.check_rc(rc, "nmb_ce_forward_fused")
    return lse, accum


def ce_bwd(logits, target, vocab_start: int, ignore_index: int, lse, gscale, out: Optional[torch.Tensor] = None):
    rows, vloc = logits.shape
    if out is None:
        out = torch.empty_like(logits)
    rc = native.lib().nmb_ce_bwd(native.ptr(logits), c_ll(logits.stride(0)), native.ptr(target), c_int(vocab_start),
                                 c_int(vloc), c_int(ignore_index), native.ptr(lse), native.ptr(gscale), native.ptr(out),
                                 c_ll(out.stride(0)), c_int(rows), native.stream_ptr(logits.device))
    native.check_rc(rc, "nmb_ce_bwd")
    return out


# -------------------------------------------------------------- embedding --
def embedding_fwd(ids, positions, tok_w, pos_w, vocab_start: int) -> torch.Tensor:
    n = ids.numel()
    vloc, h = tok_w.shape
    out = torch.empty((*ids.shape, h), dtype=torch.bfloat16, device=tok_w.device)
    rc = native.lib().nmb_embedding_fwd(native.ptr(ids), native.ptr(positions), native.ptr(tok_w), native.ptr(pos_w),
                                        native.ptr(out), c_int(n), c_int(h), c_int(vocab_start), c_int(vloc),
                                        native.stream_ptr(tok_w.device))
    native.check_rc(rc, "nmb_embedding_fwd")
    return out


def embedding_bwd(ids, positions, dy, dtok, dpos, vocab_start: int) -> None:
    """Scatter-adds ``dy`` rows into ``dtok`` (owned ids) and ``dpos``; both accumulate in place."""
    dy = _bf16(dy)
    h = dy.shape[-1]
    vloc = dtok.shape[0] if dtok is not None else 0
    rc = native.lib().nmb_embedding_bwd(native.ptr(ids), native.ptr(positions), native.ptr(dy), native.ptr(dtok),
                                        native.ptr(dpos), c_int(ids.numel()), c_int(h), c_int(vocab_start),
                                        c_int(vloc), native.stream_ptr(dy.device))
    native.check_rc(rc, "nmb_embedding_bwd")


# ------------------------------------------------------------ activations --
def gelu_fwd(x):
    x = _bf16(x)
    y = torch.empty_like(x)
    native.check_rc(native.lib().nmb_gelu_fwd(native.ptr(x), native.ptr(y), c_ll(x.numel()),
                                              native.stream_ptr(x.device)), "nmb_gelu_fwd")
    return y


def gelu_bwd(x, dy):
    x, dy = _bf16(x), _bf16(dy)
    dx = torch.empty_like(x)
    native.check_rc(native.lib().nmb_gelu_bwd(native.ptr(x), native.ptr(dy), native.ptr(dx), c_ll(x.numel()),
                                              native.stream_ptr(x.device)), "nmb_gelu_bwd")
    return dx


def swiglu_fwd(x):
    x = _bf16(x)
    f = x.shape[-1] // 2
    rows = x.numel() // (2 * f)
    y = torch.empty((*x.shape[:-1], f), dtype=torch.bfloat16, device=x.device)
    native.check_rc(native.lib().nmb_swiglu_fwd(native.ptr(x), native.ptr(y), c_ll(rows), c_int(f),
                                                native.stream_ptr(x.device)), "nmb_swiglu_fwd")
    return y


def swiglu_bwd(x, dy):
    x, dy = _bf16(x), _bf16(dy)
    f = x.shape[-1] // 2
    rows = x.numel() // (2 * f)
    dx = torch.empty_like(x)
    native.check_rc(native.lib().nmb_swiglu_bwd(native.ptr(x), native.ptr(dy), native.ptr(dx), c_ll(rows), c_int(f),
                                                native.stream_ptr(x.device)), "nmb_swiglu_bwd")
    return dx


def rope_inplace(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, sign: float) -> None:
    """Rotate interleaved pairs of a ``[B, S, heads, d]`` view in place."""
    b, s, heads, d = x.shape
    assert x.stride(3) == 1 and positions.is_contiguous()
    rc = native.lib().nmb_rope(native.ptr(x), c_ll(x.stride(0)), c_ll(x.stride(1)), c_ll(x.stride(2)),
                               native.ptr(positions), native.ptr(inv_freq), c_int(b), c_int(s), c_int(heads),
                               c_int(d), c_float(sign), native.stream_ptr(x.device))
    native.check_rc(rc, "nmb_rope")
