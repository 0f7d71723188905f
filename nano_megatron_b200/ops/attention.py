"""Causal flash attention (``csrc/attention_tcgen05.cu``) as an autograd op.

Tensors are ``[B, S, heads, d]`` *views* with a contiguous last dimension and
arbitrary other strides, so the packed output of a fused QKV projection is
consumed in place.  The key/value side may be given as a list of chunks (one
per context-parallel rank, possibly peer-memory tensors); chunk ``c`` covers
global key positions ``[c*chunk_len, (c+1)*chunk_len)`` and the query rows
start at global position ``q_pos0``.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import native


class _Tensor4(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_longlong),
                ("stride_s", ctypes.c_longlong), ("stride_h", ctypes.c_longlong)]


def _desc(t: torch.Tensor) -> _Tensor4:
    assert t.dim() == 4 and t.stride(3) == 1 and t.dtype == torch.bfloat16
    assert t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:3] if s != 0)
    return _Tensor4(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _desc_array(ts: Sequence[torch.Tensor]):
    arr = (_Tensor4 * len(ts))()
    for i, t in enumerate(ts):
        arr[i] = _desc(t)
    return arr


def _visible_kv_tiles(sq: int, q_pos0: int, skv_total: int) -> int:
    last = q_pos0 + sq - 1
    return min((last + 128) // 128, (skv_total + 127) // 128)


def attn_fwd(q, k_chunks, v_chunks, scale: float, q_pos0: int = 0):
    b, sq, hq, d = q.shape
    chunk_len, hkv = k_chunks[0].shape[1], k_chunks[0].shape[2]
    out = torch.empty((b, sq, hq, d), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
    qd, od = _desc(q), _desc(out)
    rc = native.lib().nmb_attn_fwd(
        ctypes.byref(qd), _desc_array(k_chunks), _desc_array(v_chunks), ctypes.c_int(len(k_chunks)),
        ctypes.c_int(chunk_len), ctypes.byref(od), native.ptr(lse), ctypes.c_int(b), ctypes.c_int(hq),
        ctypes.c_int(hkv), ctypes.c_int(sq), ctypes.c_int(d), ctypes.c_int(q_pos0),
        ctypes.c_float(scale), native.ptr(native.status_word(q.device)), native.stream_ptr(q.device))
    native.check_rc(rc, "nmb_attn_fwd")
    return out, lse


def attn_bwd(q, k_chunks, v_chunks, out, dout, lse, scale: float, q_pos0: int = 0,
             dk_chunks: Optional[Sequence[torch.Tensor]] = None,
             dv_chunks: Optional[Sequence[torch.Tensor]] = None,
             dq: Optional[torch.Tensor] = None, rope=None):
    """Returns ``(dq, dk_chunks, dv_chunks)``.  ``dk_chunks[c]`` receives this
    rank's contribution to chunk ``c``; rows of chunks the queries cannot see
    are left untouched (callers pass zero-filled or freshly visible buffers).
    ``dq`` / ``dk_chunks`` / ``dv_chunks`` may be strided views (for instance
    slices of one packed dQKV buffer); they are written in place.  With
    ``rope`` (a ``RopeSpec``: q and k were rotated by the projection's epilogue)
    dq and dk come back un-rotated, i.e. as gradients of the projection output;
    that needs a single key chunk as long as the query sequence."""
    b, sq, hq, d = q.shape
    chunk_len, hkv = k_chunks[0].shape[1], k_chunks[0].shape[2]
    n_chunks = len(k_chunks)
    if dout.stride(3) != 1:
        dout = dout.contiguous()
    if dq is None:
        dq = torch.empty((b, sq, hq, d), dtype=torch.bfloat16, device=q.device)
    if dk_chunks is None:
        # every key row is visible to some query: the kernel writes all of dK / dV
        covered = n_chunks == 1 and q_pos0 + sq >= chunk_len
        make = torch.empty if covered else torch.zeros
        dk_chunks = [make((b, chunk_len, hkv, d), dtype=torch.bfloat16, device=q.device) for _ in range(n_chunks)]
        dv_chunks = [make((b, chunk_len, hkv, d), dtype=torch.bfloat16, device=q.device) for _ in range(n_chunks)]
    delta = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
    dq_acc = torch.empty((b, sq, hq, d), dtype=torch.float32, device=q.device)
    n_tiles = _visible_kv_tiles(sq, q_pos0, chunk_len * n_chunks)
    qd, od, dod, dqd = _desc(q), _desc(out), _desc(dout), _desc(dq)
    rc = native.lib().nmb_attn_bwd(
        ctypes.byref(qd), _desc_array(k_chunks), _desc_array(v_chunks), ctypes.c_int(n_chunks),
        ctypes.c_int(chunk_len), ctypes.byref(od), ctypes.byref(dod), native.ptr(lse), native.ptr(delta),
        native.ptr(dq_acc), ctypes.byref(dqd), _desc_array(dk_chunks), _desc_array(dv_chunks),
        ctypes.c_int(b), ctypes.c_int(hq), ctypes.c_int(hkv), ctypes.c_int(sq), ctypes.c_int(d),
        ctypes.c_int(q_pos0), ctypes.c_int(n_tiles), ctypes.c_float(scale),
        native.ptr(rope.table if rope is not None else None),
        native.ptr(rope.positions if rope is not None else None),
        native.ptr(native.status_word(q.device)), native.stream_ptr(q.device))
    native.check_rc(rc, "nmb_attn_bwd")
    return dq, list(dk_chunks), list(dv_chunks)


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        out, lse = attn_fwd(q, [k], [v], scale, 0)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = attn_bwd(q, [k], [v], out, dout, lse, ctx.scale, 0)
        return dq, dk[0], dv[0], None


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """Causal attention over ``[B, S, heads, d]`` views; returns ``[B, S, Hq, d]``."""
    return _FlashAttention.apply(q, k, v, float(scale))


def _split_packed(qkv: torch.Tensor, hq: int, hkv: int, d: int):
    b, s, _ = qkv.shape
    q = qkv[..., : hq * d].view(b, s, hq, d)
    k = qkv[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
    v = qkv[..., (hq + hkv) * d:].view(b, s, hkv, d)
    return q, k, v


class _FlashAttentionPacked(torch.autograd.Function):
    """Attention straight from / to the packed ``[B, S, (Hq + 2 Hkv) d]`` tensor of a
    fused QKV projection: forward reads its three slices in place, backward has
    the kernels write dQ, dK and dV into the slices of ONE gradient buffer, so no
    slice-gradient zero-fill / copy / add kernels run around the attention."""

    @staticmethod
    def forward(ctx, qkv, hq, hkv, d, scale, rope=None):
        q, k, v = _split_packed(qkv, hq, hkv, d)
        out, lse = attn_fwd(q, [k], [v], scale, 0)
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (hq, hkv, d, scale, rope)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        hq, hkv, d, scale, rope = ctx.meta
        q, k, v = _split_packed(qkv, hq, hkv, d)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = _split_packed(dqkv, hq, hkv, d)
        attn_bwd(q, [k], [v], out, dout, lse, scale, 0, dk_chunks=[dk], dv_chunks=[dv], dq=dq, rope=rope)
        return dqkv, None, None, None, None, None


def flash_attention_packed(qkv: torch.Tensor, hq: int, hkv: int, d: int, scale: float, rope=None) -> torch.Tensor:
    """Causal attention over a packed, contiguous ``[B, S, (Hq + 2 Hkv) d]`` tensor
    (query heads, then key heads, then value heads); returns ``[B, S, Hq, d]``.

    ``rope``: the q and k slices were rotated by the epilogue of the projection
    that produced ``qkv`` (``linear(..., rope=spec)``).  The forward pass is the
    same; the backward pass un-rotates dq and dk inside its last kernel, so the
    gradient returned for ``qkv`` is the gradient of the projection's
    *un-rotated* output and the projection's backward stays a plain linear
    backward.  The two must be used together."""
    assert qkv.dim() == 3 and qkv.is_contiguous() and qkv.shape[-1] == (hq + 2 * hkv) * d
    return _FlashAttentionPacked.apply(qkv, hq, hkv, d, float(scale), rope)


class _SplitPacked(torch.autograd.Function):
    """``qkv -> (q, k, v)`` views whose gradients are joined by one concatenation
    kernel instead of three zero-fills, three strided copies and two adds."""

    @staticmethod
    def forward(ctx, qkv, hq, hkv, d):
        ctx.meta = (hq, hkv, d)
        return _split_packed(qkv, hq, hkv, d)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        b, s = dq.shape[0], dq.shape[1]
        hq, hkv, d = ctx.meta
        width = (hq + 2 * hkv) * d
        packed = (dq.stride() == (s * width, width, d, 1) and dk.stride() == dq.stride() and dv.stride() == dq.stride()
                  and dk.data_ptr() == dq.data_ptr() + 2 * hq * d and dv.data_ptr() == dk.data_ptr() + 2 * hkv * d
                  and dq.dtype == torch.bfloat16)
        if packed:
            # the three gradients already are the slices of one packed buffer: hand that buffer back
            return dq.as_strided((b, s, width), (s * width, width, 1)), None, None, None
        return torch.cat([dq.reshape(b, s, -1), dk.reshape(b, s, -1), dv.reshape(b, s, -1)], dim=-1), None, None, None


def split_packed_qkv(qkv: torch.Tensor, hq: int, hkv: int, d: int):
    """Differentiable ``[B, S, (Hq + 2 Hkv) d] -> q, k, v`` views (``[B, S, heads, d]``)."""
    return _SplitPacked.apply(qkv, hq, hkv, d)


def attention_supported(d: int) -> bool:
    return d in (64, 96, 128)
