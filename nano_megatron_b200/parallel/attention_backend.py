"""Attention backend resolution and the three attention entry points.

Names and tensor conventions (``[B, heads, S, d]`` in and out) follow the
reference (nano_megatron/parallel/attention_backend.py:22-635).  ``"flash"``
here is this package's own tcgen05 kernel (``csrc/attention_tcgen05.cu``), not
the flash-attn package: it needs a CUDA device, bf16 and head_dim 64/96/128.
The context-parallel entry point keeps the reference's name
``flash_ring_causal_attention`` although, as there, it is "all keys visible to
every rank" rather than a P2P ring: the kernel walks the K/V chunks of the
ranks ``<= cp_rank`` (gathered with one all-gather each, or read in place from
peer memory when a symmetric-memory workspace is supplied) and merges the
partial softmaxes in registers.
"""
from __future__ import annotations

from typing import Any, Literal, Optional

import torch
from torch import Tensor

from ..distributed.backend import CommBackend
from ..ops import native
from .context_parallel import causal_attn_scores_cp

AttentionBackendName = Literal["flash", "unfused"]
RequestedAttentionBackend = Literal["auto", "flash", "unfused"]

_FLASH_DTYPES = (torch.bfloat16,)


def flash_attn_available() -> bool:
    """True when the in-tree kernel library has been built."""
    return native.available()


def resolve_attention_backend(*, requested: str, dtype: torch.dtype, device: torch.device,
                              return_activations: bool = False) -> AttentionBackendName:
    if return_activations:
        return "unfused"
    if requested not in ("auto", "flash", "unfused"):
        raise ValueError(f"requested must be one of 'auto', 'flash', 'unfused'; got {requested!r}")
    if requested == "unfused":
        return "unfused"
    device = torch.device(device)
    ok = device.type == "cuda" and dtype in _FLASH_DTYPES and flash_attn_available()
    if requested == "auto":
        return "flash" if ok else "unfused"
    if ok:
        return "flash"
    why = []
    if device.type != "cuda":
        why.append(f"device must be CUDA (got {device})")
    if dtype not in _FLASH_DTYPES:
        why.append(f"dtype must be bfloat16 (got {dtype})")
    if not flash_attn_available():
        why.append("the kernel library is not built")
    raise RuntimeError("attn_backend='flash' requires CUDA, bf16 and the built kernel library; " + "; ".join(why))


def _check_qkv(q: Tensor, k: Tensor, v: Tensor) -> None:
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError(f"q, k, v must be 4D [B,H,S,D]; got q={tuple(q.shape)}, k={tuple(k.shape)}, v={tuple(v.shape)}")
    if k.shape != v.shape:
        raise ValueError(f"k and v must share shape; got k={tuple(k.shape)}, v={tuple(v.shape)}")
    if q.shape[0] != k.shape[0] or q.shape[3] != k.shape[3]:
        raise ValueError(f"q/k batch and head_dim must match; got q={tuple(q.shape)}, k={tuple(k.shape)}")


def unfused_causal_attention(q: Tensor, k: Tensor, v: Tensor, *, scale: float,
                             query_start: Optional[int] = None) -> Tensor:
    """scores -> softmax -> @V.  With ``query_start`` the queries are a shard
    whose first row sits at that global position (context parallel)."""
    from ..reference.layers import causal_attn_scores, softmax_last

    _check_qkv(q, k, v)
    if q.shape[1] != k.shape[1]:
        raise ValueError(f"q/k heads must match; got q={tuple(q.shape)}, k={tuple(k.shape)}")
    if query_start is None:
        if q.size(2) != k.size(2):
            raise ValueError("query_start is required when q and k sequence lengths differ")
        scores = causal_attn_scores(q, k, scale=scale)
    else:
        if query_start < 0 or query_start + q.size(2) > k.size(2):
            raise ValueError(f"query_start ({query_start}) + S_q ({q.size(2)}) exceeds S_k ({k.size(2)})")
        scores = causal_attn_scores_cp(q, k, scale=scale, query_start=query_start)
    return torch.matmul(softmax_last(scores), v)


def _require_flash(q: Tensor, dropout_p: float) -> None:
    if q.device.type != "cuda":
        raise RuntimeError(f"flash attention requires a CUDA device, got {q.device}")
    if q.dtype not in _FLASH_DTYPES:
        raise RuntimeError(f"flash attention requires bfloat16, got {q.dtype}")
    if q.shape[-1] not in (64, 96, 128):
        raise RuntimeError(f"flash attention supports head_dim 64/96/128, got {q.shape[-1]}")
    if dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not implemented in the tcgen05 kernel")


def flash_causal_attention(q: Tensor, k: Tensor, v: Tensor, *, scale: float, dropout_p: float = 0.0) -> Tensor:
    """Fused causal attention; ``k``/``v`` may have fewer (grouped) heads."""
    from ..ops.attention import flash_attention

    _check_qkv(q, k, v)
    _require_flash(q, dropout_p)
    out = flash_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale)
    return out.transpose(1, 2)


def _online_softmax_combine(out_a: Tensor, lse_a: Tensor, out_b: Tensor, lse_b: Tensor) -> tuple[Tensor, Tensor]:
    """Merge two partial attention results over disjoint key sets.

    ``out_*`` are normalised partial outputs, ``lse_*`` the ``[B, h, S]`` log-sum-exp of
    their scores; fp32 arithmetic.  The outputs may be ``[B, S, h, d]`` (the layout of this
    package's kernels) or ``[B, h, S, d]`` (the reference's helper,
    nano_megatron/parallel/attention_backend.py:227-270); the layout is read off the shapes
    and ``[B, S, h, d]`` is assumed when ``h == S`` makes them indistinguishable.
    """
    if out_a.shape != out_b.shape or lse_a.shape != lse_b.shape:
        raise ValueError(f"partial results must share shapes; got {tuple(out_a.shape)} vs {tuple(out_b.shape)} "
                         f"and {tuple(lse_a.shape)} vs {tuple(lse_b.shape)}")
    lse_a, lse_b = lse_a.float(), lse_b.float()
    top = torch.maximum(lse_a, lse_b)
    wa, wb = torch.exp(lse_a - top), torch.exp(lse_b - top)
    total = wa + wb
    lse = top + torch.log(total)
    ca, cb = wa / total, wb / total
    heads_first = tuple(out_a.shape[1:3]) == tuple(lse.shape[1:3]) and out_a.shape[1] != out_a.shape[2]
    if not heads_first:
        ca, cb = ca.transpose(1, 2), cb.transpose(1, 2)
    return (out_a.float() * ca.unsqueeze(-1) + out_b.float() * cb.unsqueeze(-1)).to(out_a.dtype), lse


class _FlashChunkedCPCausalAttention(torch.autograd.Function):
    """Local queries against the K/V chunks of ranks ``0..cp_rank``.

    ``k_chunks`` / ``v_chunks`` are ``cp_size`` tensors ``[B, S_loc, h_kv, d]``
    (views of a gathered buffer or peer-memory tensors).  The backward produces
    this rank's contribution to every chunk's dK/dV; chunks in the causal
    future stay zero.
    """

    @staticmethod
    def forward(ctx: Any, q: Tensor, k_all: Tensor, v_all: Tensor, scale: float, cp_rank: int, cp_size: int):
        from ..ops.attention import attn_fwd

        s_loc = q.shape[1]
        ks = [k_all[:, c * s_loc:(c + 1) * s_loc] for c in range(cp_size)]
        vs = [v_all[:, c * s_loc:(c + 1) * s_loc] for c in range(cp_size)]
        out, lse = attn_fwd(q, ks, vs, scale, q_pos0=cp_rank * s_loc)
        ctx.save_for_backward(q, k_all, v_all, out, lse)
        ctx.meta = (scale, cp_rank, cp_size)
        return out

    @staticmethod
    def backward(ctx: Any, dout: Tensor):
        from ..ops.attention import attn_bwd

        q, k_all, v_all, out, lse = ctx.saved_tensors
        scale, cp_rank, cp_size = ctx.meta
        s_loc = q.shape[1]
        ks = [k_all[:, c * s_loc:(c + 1) * s_loc] for c in range(cp_size)]
        vs = [v_all[:, c * s_loc:(c + 1) * s_loc] for c in range(cp_size)]
        dk_all, dv_all = torch.zeros_like(k_all), torch.zeros_like(v_all)
        dks = [dk_all[:, c * s_loc:(c + 1) * s_loc] for c in range(cp_size)]
        dvs = [dv_all[:, c * s_loc:(c + 1) * s_loc] for c in range(cp_size)]
        dq, _, _ = attn_bwd(q, ks, vs, out, dout, lse, scale, q_pos0=cp_rank * s_loc, dk_chunks=dks, dv_chunks=dvs)
        return dq, dk_all, dv_all, None, None, None


def _flash_chunked_cp_causal_attention(q: Tensor, k_full: Tensor, v_full: Tensor, *, scale: float, cp_rank: int,
                                       cp_size: int) -> Tensor:
    """``q`` ``[B,h,S_loc,d]`` against full ``k``/``v`` ``[B,h_kv,S,d]``; usable
    in one process to emulate any ``cp_rank``."""
    out = _FlashChunkedCPCausalAttention.apply(q.transpose(1, 2), k_full.transpose(1, 2), v_full.transpose(1, 2),
                                               scale, cp_rank, cp_size)
    return out.transpose(1, 2)


def flash_ring_causal_attention(q: Tensor, k: Tensor, v: Tensor, *, scale: float, cp_group: Any, cp_rank: int,
                                cp_size: int, backend: CommBackend, dropout_p: float = 0.0) -> Tensor:
    """Context-parallel fused attention over contiguous sequence shards."""
    from .context_parallel import gather_from_context_parallel_region

    _check_qkv(q, k, v)
    if cp_size > 1 and dropout_p != 0.0:
        raise NotImplementedError("attention dropout is not supported with context-parallel flash attention")
    if cp_size == 1:
        return flash_causal_attention(q, k, v, scale=scale, dropout_p=dropout_p)
    _require_flash(q, dropout_p)
    if q.size(2) % 128 != 0:
        raise ValueError(f"context-parallel flash attention needs S_local % 128 == 0, got {q.size(2)}")
    k_full = gather_from_context_parallel_region(k, cp_group, backend, cp_rank, cp_size, seq_dim=2,
                                                 grad_op="reduce_scatter")
    v_full = gather_from_context_parallel_region(v, cp_group, backend, cp_rank, cp_size, seq_dim=2,
                                                 grad_op="reduce_scatter")
    return _flash_chunked_cp_causal_attention(q, k_full, v_full, scale=scale, cp_rank=cp_rank, cp_size=cp_size)
