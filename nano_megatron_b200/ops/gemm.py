"""Python entry point of the tcgen05 bf16 GEMM (``csrc/gemm_tcgen05.cu``).

``gemm_bf16`` computes ``C[M,N] = epilogue(alpha * A @ B^T)`` where the logical
operands are ``A[M,K]`` and ``B[N,K]``.  With ``a_mn`` / ``b_mn`` the tensor
passed in is the *transpose* of the logical operand (``[K,M]`` / ``[K,N]``), read
in place by the kernel as an MN-major operand, so dgrad and wgrad need no
transposed copies.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import native

EPI_PLAIN, EPI_GELU, EPI_DGELU, EPI_ROPE, EPI_SWIGLU, EPI_DSWIGLU = 0, 1, 2, 3, 4, 5


class _EpilogueExtra(ctypes.Structure):
    _fields_ = [("rope_table", ctypes.c_void_p), ("rope_pos", ctypes.c_void_p), ("rope_cols", ctypes.c_int),
                ("rope_half", ctypes.c_int), ("swiglu_f", ctypes.c_int)]


@dataclass
class RopeSpec:
    """Rotary embedding applied by a GEMM epilogue (and undone by the attention
    backward): ``table[p, i] = (cos, sin)`` of position ``p`` times inverse
    frequency ``i`` (fp32, ``[positions, head_dim / 2, 2]``), ``positions`` the
    position of every output row (int64, ``rows`` long when flattened), and the
    number of leading output columns that hold rotated heads (q and k)."""

    table: torch.Tensor
    positions: torch.Tensor
    rope_cols: int

    @property
    def half(self) -> int:
        return self.table.shape[1]

    @staticmethod
    def make_table(inv_freq: torch.Tensor, max_positions: int) -> torch.Tensor:
        ang = torch.outer(torch.arange(max_positions, device=inv_freq.device, dtype=torch.float32),
                          inv_freq.to(torch.float32))
        return torch.stack([ang.cos(), ang.sin()], dim=-1).contiguous()


def epilogue_extra(rope: Optional[RopeSpec] = None, swiglu_f: int = 0):
    """ctypes argument for the optional epilogue parameters (``None`` when unused)."""
    if rope is None and not swiglu_f:
        return None
    ex = _EpilogueExtra()
    if rope is not None:
        assert rope.table.dtype == torch.float32 and rope.table.is_contiguous()
        assert rope.positions.dtype == torch.long and rope.positions.is_contiguous()
        ex.rope_table, ex.rope_pos = rope.table.data_ptr(), rope.positions.data_ptr()
        ex.rope_cols, ex.rope_half = int(rope.rope_cols), int(rope.half)
    ex.swiglu_f = int(swiglu_f)
    return ex


def _as_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    if t.stride(-1) != 1:
        t = t.contiguous()
    return t


def gemm_supported(k: int, lda: int, ldb: int, ldc: int) -> bool:
    """TMA needs 16-byte row pitches; the vector epilogue 16-byte rows of C."""
    return k > 0 and lda % 8 == 0 and ldb % 8 == 0 and ldc % 8 == 0


def gemm_bf16(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    mode: int = EPI_PLAIN,
    aux_in: Optional[torch.Tensor] = None,
    aux_out: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    out_dtype: torch.dtype = torch.bfloat16,
    alpha: float = 1.0,
    rope: Optional[RopeSpec] = None,
    swiglu_f: int = 0,
) -> torch.Tensor:
    a = _as_2d(a)
    b = _as_2d(b)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "bf16 operands only"
    if a_mn:
        k, m = a.shape
    else:
        m, k = a.shape
    if b_mn:
        kb, n = b.shape
    else:
        n, kb = b.shape
    if k != kb:
        raise ValueError(f"reduction dims differ: {k} vs {kb}")
    # SwiGLU: the B rows are [gate; up] (n = 2F) and C is [m, F]; its backward
    # epilogue turns d(act) [m, F] into [d gate | d up] = [m, 2F]
    out_cols = {EPI_SWIGLU: n // 2, EPI_DSWIGLU: 2 * n}.get(mode, n)
    if out is None:
        out = torch.empty((m, out_cols), dtype=out_dtype, device=a.device)
    else:
        assert out.shape == (m, out_cols) and out.stride(1) == 1
    if mode == EPI_SWIGLU:
        assert aux_out is not None
        swiglu_f = n // 2
    elif mode == EPI_DSWIGLU:
        assert aux_in is not None
        swiglu_f = n
    if mode == EPI_GELU and aux_out is None:
        aux_out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    if residual is not None:
        residual = _as_2d(residual)
    aux = aux_out if mode in (EPI_GELU, EPI_SWIGLU) else aux_in
    if aux is not None:
        aux = _as_2d(aux)
    ld_aux = aux.stride(0) if aux is not None else 0
    status = native.status_word(a.device)
    extra = epilogue_extra(rope if mode == EPI_ROPE else None, swiglu_f)
    rc = native.lib().nmb_gemm_bf16(
        native.ptr(a), ctypes.c_int(a.stride(0)), ctypes.c_int(int(a_mn)),
        native.ptr(b), ctypes.c_int(b.stride(0)), ctypes.c_int(int(b_mn)),
        native.ptr(out), ctypes.c_int(out.stride(0)),
        ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k),
        native.ptr(bias), native.ptr(residual),
        ctypes.c_int(residual.stride(0) if residual is not None else 0),
        native.ptr(aux if mode in (EPI_GELU, EPI_SWIGLU) else None),
        native.ptr(aux if mode in (EPI_DGELU, EPI_DSWIGLU) else None),
        ctypes.c_int(ld_aux), ctypes.c_int(mode), ctypes.c_int(int(accumulate)),
        ctypes.c_int(int(out.dtype == torch.float32)), ctypes.c_float(alpha),
        ctypes.byref(extra) if extra is not None else None,
        native.ptr(status), native.stream_ptr(a.device),
    )
    native.check_rc(rc, "nmb_gemm_bf16")
    return out
