"""Autograd-level ops used by the parallel layers and models.

Every function has two implementations behind one name:

* CUDA + bf16 tensors  -> the sm_100a kernels of this package (tcgen05 GEMM
  with fused epilogues, fused norm / CE / embedding kernels), with hand-written
  backward passes;
* anything else (CPU, fp32) -> the plain PyTorch expression of the same maths,
  which is what the oracle and the Gloo tests run.

There is no third path and no silent fallback on a GPU: bf16 CUDA tensors
always go to the native kernels (a missing library raises).

Gradient buffers.  A parameter may carry ``main_grad`` -- a persistent tensor
of its own shape (a view into a DDP bucket or a model-wide flat buffer).  The
weight-gradient GEMM, the bias reduction and the embedding scatter then
accumulate straight into it, return no gradient to autograd, and announce
completion through ``param._nmb_grad_ready()`` when that attribute exists.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.nn.functional as F
from torch import Tensor

from . import kernels
from .gemm import (EPI_DGELU, EPI_DSWIGLU, EPI_GELU, EPI_PLAIN, EPI_ROPE, EPI_SWIGLU, RopeSpec, gemm_bf16,
                   gemm_supported)


def use_native(t: Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


# First write of a step overwrites.  A gradient buffer need not be zeroed when the
# first kernel that writes it in a step stores instead of adding: the owner of the
# buffers (the data-parallel wrapper) sets ``param._nmb_overwrite_next`` in place
# of the memset, and the first delivery below clears it.  To learn which parameters
# qualify it traces one backward pass: every writer of a ``main_grad`` reports
# here, "direct" when it can overwrite, "other" when it can only add (scatter-add,
# autograd accumulation); only parameters whose FIRST write was "direct" qualify.
_GRAD_TRACES: list[dict[int, str]] = []


def note_grad_write(param: Optional[Tensor], direct: bool) -> None:
    if param is None:
        return
    for trace in _GRAD_TRACES:
        trace.setdefault(id(param), "direct" if direct else "other")


def take_overwrite(param: Optional[Tensor]) -> bool:
    """True (once) when the next write to ``param.main_grad`` must overwrite it."""
    if param is not None and getattr(param, "_nmb_overwrite_next", False):
        param._nmb_overwrite_next = False
        return True
    return False


def _deliver_grad(param: Optional[Tensor], compute, *, shape_like: Optional[Tensor] = None):
    """Run ``compute(out, accumulate)``; returns the grad for autograd or None
    when it was written into ``param.main_grad`` (added, or stored when the
    buffer's owner asked for the first write of the step to overwrite)."""
    main = getattr(param, "main_grad", None) if param is not None else None
    if main is not None and getattr(param, "_nmb_sp_replicated", False):
        main = None  # its TP gradient hook only runs on the autograd path
    if main is not None:
        note_grad_write(param, True)
        compute(main, not take_overwrite(param))
        ready = getattr(param, "_nmb_grad_ready", None)
        if ready is not None:
            ready()
        return None
    return compute(None, False)


# ------------------------------------------------------------------ linear --
class _LinearFn(torch.autograd.Function):
    """y = act(x W^T + b) (+ residual) on the tcgen05 GEMM."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Optional[Tensor], residual: Optional[Tensor], gelu: bool,
                rope: Optional[RopeSpec] = None, out: Optional[Tensor] = None):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1 or (x2.stride(0) % 8) != 0:
            x2 = x2.contiguous()
        n = weight.shape[0]
        res2 = residual.reshape(-1, n) if residual is not None else None
        pre = None
        if gelu:
            pre = torch.empty((x2.shape[0], n), dtype=torch.bfloat16, device=x.device)
            y = gemm_bf16(x2, weight, bias=bias, mode=EPI_GELU, aux_out=pre)
        elif rope is not None:
            # q and k heads leave the projection already rotated; the attention
            # backward hands back the gradient of the un-rotated output, so the
            # backward below is the plain linear one
            y = gemm_bf16(x2, weight, bias=bias, mode=EPI_ROPE, rope=rope,
                          out=out.view(-1, n) if out is not None else None)
        else:
            # ``out``: a caller-provided destination (e.g. symmetric memory that peers read)
            y = gemm_bf16(x2, weight, bias=bias, residual=res2, mode=EPI_PLAIN,
                          out=out.view(-1, n) if out is not None else None)
        ctx.save_for_backward(x2, weight, pre)
        ctx.has_bias = bias is not None
        ctx.has_res = residual is not None
        ctx.params = (weight, bias)
        ctx.in_shape = x.shape
        return y.view(*x.shape[:-1], n)

    @staticmethod
    def backward(ctx, dy: Tensor):
        x2, weight, pre = ctx.saved_tensors
        w_param, b_param = ctx.params
        n = weight.shape[0]
        dy2 = dy.reshape(-1, n)
        if dy2.stride(-1) != 1 or (dy2.stride(0) % 8) != 0:
            dy2 = dy2.contiguous()
        d_res = dy if ctx.has_res else None
        dz = kernels.gelu_bwd(pre, dy2) if pre is not None else dy2
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm_bf16(dz, weight, b_mn=True).view(ctx.in_shape)
        dw = None
        if ctx.needs_input_grad[1]:
            dw = _deliver_grad(
                w_param,
                lambda out, acc: gemm_bf16(dz, x2, a_mn=True, b_mn=True, out=out, accumulate=acc),
            )
        db = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = _deliver_grad(b_param, lambda out, acc: kernels.col_sum(dz, out=out, accumulate=acc))
        return dx, dw, db, d_res, None, None, None


def _rows(t: Tensor, width: int) -> Tensor:
    t2 = t.reshape(-1, width)
    if t2.stride(-1) != 1 or (t2.stride(0) % 8) != 0:
        t2 = t2.contiguous()
    return t2


class _LinearActSplitFn(torch.autograd.Function):
    """First MLP GEMM: returns the pre-activation (differentiable) and its
    activation (a side output written by the same epilogue).  ``act`` is
    ``"gelu"`` (pre and activation both ``[.., F]``) or ``"swiglu"`` (weight rows
    ``[gate; up]``, pre ``[.., 2F]``, activation ``silu(gate) * up`` ``[.., F]``)."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Optional[Tensor], act: str):
        x2 = _rows(x, x.shape[-1])
        n = weight.shape[0]
        pre = torch.empty((x2.shape[0], n), dtype=torch.bfloat16, device=x.device)
        out = gemm_bf16(x2, weight, bias=bias, mode=EPI_SWIGLU if act == "swiglu" else EPI_GELU, aux_out=pre)
        ctx.save_for_backward(x2, weight)
        ctx.params = (weight, bias)
        ctx.in_shape = x.shape
        out = out.view(*x.shape[:-1], out.shape[-1])
        ctx.mark_non_differentiable(out)
        # no zero-filled gradient tensor for the non-differentiable side output
        ctx.set_materialize_grads(False)
        return pre.view(*x.shape[:-1], n), out

    @staticmethod
    def backward(ctx, dpre: Optional[Tensor], _dact):
        x2, weight = ctx.saved_tensors
        w_param, b_param = ctx.params
        if dpre is None:
            return None, None, None, None
        dz = _rows(dpre, weight.shape[0])
        dx = gemm_bf16(dz, weight, b_mn=True).view(ctx.in_shape) if ctx.needs_input_grad[0] else None
        dw = _deliver_grad(w_param, lambda out, acc: gemm_bf16(dz, x2, a_mn=True, b_mn=True, out=out, accumulate=acc))
        db = None
        if b_param is not None:
            db = _deliver_grad(b_param, lambda out, acc: kernels.col_sum(dz, out=out, accumulate=acc))
        return dx, dw, db, None


class _LinearFromActFn(torch.autograd.Function):
    """Second MLP GEMM.  Its input is ``act(pre)`` (already computed); the
    gradient it returns is with respect to ``pre``: GELU' / the SwiGLU backward
    is applied in the epilogue of the dgrad GEMM, so no separate
    activation-backward kernel runs."""

    @staticmethod
    def forward(ctx, pre: Tensor, act_t: Tensor, weight: Tensor, bias: Optional[Tensor], residual: Optional[Tensor],
                act: str):
        k = act_t.shape[-1]
        a2 = _rows(act_t, k)
        n = weight.shape[0]
        res2 = residual.reshape(-1, n) if residual is not None else None
        y = gemm_bf16(a2, weight, bias=bias, residual=res2)
        ctx.save_for_backward(_rows(pre, pre.shape[-1]), a2, weight)
        ctx.params = (weight, bias)
        ctx.meta = (residual is not None, pre.shape, act)
        return y.view(*act_t.shape[:-1], n)

    @staticmethod
    def backward(ctx, dy: Tensor):
        pre2, a2, weight = ctx.saved_tensors
        w_param, b_param = ctx.params
        has_res, pre_shape, act = ctx.meta
        dy2 = _rows(dy, weight.shape[0])
        dpre = gemm_bf16(dy2, weight, b_mn=True, mode=EPI_DSWIGLU if act == "swiglu" else EPI_DGELU,
                         aux_in=pre2).view(pre_shape)
        dw = _deliver_grad(w_param, lambda out, acc: gemm_bf16(dy2, a2, a_mn=True, b_mn=True, out=out, accumulate=acc))
        db = None
        if b_param is not None:
            db = _deliver_grad(b_param, lambda out, acc: kernels.col_sum(dy2, out=out, accumulate=acc))
        return dpre, None, dw, db, (dy if has_res else None), None


def linear_gelu_split(x: Tensor, weight: Tensor, bias: Optional[Tensor]) -> tuple[Tensor, Tensor]:
    """``pre = x W^T + b`` and ``gelu(pre)`` from one GEMM (native path only)."""
    return _LinearActSplitFn.apply(x, weight, bias, "gelu")


def linear_act_split(x: Tensor, weight: Tensor, bias: Optional[Tensor], act: str) -> tuple[Tensor, Tensor]:
    """``pre = x W^T + b`` and ``act(pre)`` from one GEMM (native path only)."""
    return _LinearActSplitFn.apply(x, weight, bias, act)


def linear_from_gelu(pre: Tensor, act: Tensor, weight: Tensor, bias: Optional[Tensor],
                     residual: Optional[Tensor] = None) -> Tensor:
    """``act W^T + b (+ residual)`` where ``act = gelu(pre)``; backward flows into ``pre``."""
    return _LinearFromActFn.apply(pre, act, weight, bias, residual, "gelu")


def linear_from_act(pre: Tensor, act_t: Tensor, weight: Tensor, bias: Optional[Tensor],
                    residual: Optional[Tensor] = None, act: str = "gelu") -> Tensor:
    """``act_t W^T + b (+ residual)`` where ``act_t = act(pre)``; backward flows into ``pre``."""
    return _LinearFromActFn.apply(pre, act_t, weight, bias, residual, act)


def swiglu_epilogue_ok(weight: Tensor) -> bool:
    """The fused SwiGLU epilogue needs whole 32-column chunks of gate / up."""
    return weight.shape[0] % 64 == 0


def native_linear_ok(x: Tensor, weight: Tensor) -> bool:
    k = x.shape[-1]
    n = weight.shape[0]
    return use_native(x) and weight.dtype == torch.bfloat16 and weight.is_contiguous() and \
        gemm_supported(k, k, k, n) and n % 8 == 0


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, *, residual: Optional[Tensor] = None,
           gelu: bool = False, rope: Optional[RopeSpec] = None, out: Optional[Tensor] = None) -> Tensor:
    """``act(x @ weight.T + bias) + residual`` (``gelu`` and ``residual`` are exclusive).
    ``rope`` (native path only) rotates the leading q / k columns in the epilogue."""
    assert not (gelu and residual is not None)
    if native_linear_ok(x, weight):
        return _LinearFn.apply(x, weight, bias, residual, gelu, rope, out)
    assert rope is None and out is None, "the rotary epilogue / output buffer exist on the native path only"
    # Rows that are not multiples of 16 bytes cannot be described to TMA; such
    # (toy) shapes use the PyTorch expression below.
    y = F.linear(x, weight, bias)
    if gelu:
        from ..reference.layers import gelu_erf
        y = gelu_erf(y)
    if residual is not None:
        y = residual + y
    return y


# -------------------------------------------------------------------- norm --
def _norm_grad_targets(w_param, b_param, want_bias: bool):
    """The parameters' persistent gradient buffers when the norm backward may add
    to them directly (bf16 ``main_grad`` on every parameter involved, none of
    them reduced over the sequence-parallel group by an autograd hook)."""
    params = [w_param] + ([b_param] if want_bias else [])
    bufs = []
    for p in params:
        main = getattr(p, "main_grad", None)
        if main is None or main.dtype != torch.bfloat16 or getattr(p, "_nmb_sp_replicated", False):
            return None
        bufs.append(main)
    return (bufs[0], bufs[1] if want_bias else None), params


class _NormFn(torch.autograd.Function):
    """LayerNorm / RMSNorm.  With ``passthrough`` the input is also returned
    unchanged as a second output for the residual connection, so that backward
    receives the residual branch's gradient together with dy and adds it inside
    the dx kernel (no separate accumulation kernel)."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Optional[Tensor], eps: float, rms: bool, passthrough: bool):
        y, mean, rstd = kernels.norm_fwd(x, weight, bias, eps, rms)
        ctx.save_for_backward(x, weight, mean, rstd)
        ctx.rms = rms
        ctx.params = (weight, bias)
        ctx.passthrough = passthrough
        if passthrough:
            return y, x.view_as(x)
        return y

    @staticmethod
    def backward(ctx, dy: Optional[Tensor], dres: Optional[Tensor] = None):
        x, weight, mean, rstd = ctx.saved_tensors
        w_param, b_param = ctx.params
        want_bias = b_param is not None and not ctx.rms
        if dy is None:  # only the residual branch was used
            return dres, None, None, None, None, None
        if dres is not None and (dres.shape != x.shape or not dres.is_contiguous()):
            dres = dres.expand_as(x).contiguous()
        targets = _norm_grad_targets(w_param, b_param, want_bias)
        if targets is not None:
            bufs, params = targets
            for p in params:
                note_grad_write(p, True)
            flagged = [take_overwrite(p) for p in params]
            overwrite = all(flagged)
            if any(flagged) and not overwrite:   # never in practice: both belong to one module
                for p, f in zip(params, flagged):
                    if f:
                        p.main_grad.zero_()
            dx, _, _ = kernels.norm_bwd(dy, x, weight, mean, rstd, ctx.rms, dx_add=dres, want_bias=want_bias,
                                        grad_out=bufs, accumulate=not overwrite)
            for p in params:
                ready = getattr(p, "_nmb_grad_ready", None)
                if ready is not None:
                    ready()
            return dx, None, None, None, None, None
        dx, dw, db = kernels.norm_bwd(dy, x, weight, mean, rstd, ctx.rms, dx_add=dres, want_bias=want_bias)
        return dx, dw, db, None, None, None


def layer_norm(x: Tensor, weight: Tensor, bias: Optional[Tensor], eps: float) -> Tensor:
    if use_native(x) and x.shape[-1] % 2 == 0:
        return _NormFn.apply(x, weight, bias, eps, False, False)
    return F.layer_norm(x, (x.shape[-1],), weight=weight, bias=bias, eps=eps)


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    if use_native(x) and x.shape[-1] % 2 == 0:
        return _NormFn.apply(x, weight, None, eps, True, False)
    from ..reference.layers import rms_norm as _rms
    return _rms(x, weight, eps)


def norm_with_residual(x: Tensor, weight: Tensor, bias: Optional[Tensor], eps: float, rms: bool):
    """``(norm(x), x)`` for a pre-norm residual block: use the second value for
    the residual connection.  On the native path its gradient is folded into the
    norm's dx kernel."""
    if use_native(x) and x.shape[-1] % 2 == 0 and x.is_contiguous():
        return _NormFn.apply(x, weight, None if rms else bias, eps, rms, True)
    return (rms_norm(x, weight, eps) if rms else layer_norm(x, weight, bias, eps)), x


# ------------------------------------------------------------- activations --
class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return kernels.gelu_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return kernels.gelu_bwd(x, dy)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return kernels.swiglu_fwd(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return kernels.swiglu_bwd(x, dy)


def gelu(x: Tensor) -> Tensor:
    if use_native(x) and x.numel() % 2 == 0:
        return _GeluFn.apply(x)
    from ..reference.layers import gelu_erf
    return gelu_erf(x)


def swiglu(x: Tensor) -> Tensor:
    if use_native(x) and (x.shape[-1] // 2) % 2 == 0:
        return _SwigluFn.apply(x)
    from ..reference.layers import swiglu as _sw
    return _sw(x)


class _RopeFn(torch.autograd.Function):
    """Rotates q and k in place inside the packed projection output."""

    @staticmethod
    def forward(ctx, x: Tensor, positions: Tensor, inv_freq: Tensor):
        out = x.clone()
        kernels.rope_inplace(out, positions, inv_freq, 1.0)
        ctx.save_for_backward(positions, inv_freq)
        return out

    @staticmethod
    def backward(ctx, dy: Tensor):
        positions, inv_freq = ctx.saved_tensors
        dx = dy.clone()
        kernels.rope_inplace(dx, positions, inv_freq, -1.0)
        return dx, None, None


def rope_bshd(x: Tensor, positions: Tensor, inv_freq: Tensor) -> Tensor:
    """Rotary embedding on a ``[B, S, heads, d]`` bf16 CUDA tensor (interleaved pairs)."""
    return _RopeFn.apply(x, positions.contiguous(), inv_freq)


# --------------------------------------------------------------- embedding --
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids: Tensor, positions: Optional[Tensor], tok_w: Tensor, pos_w: Optional[Tensor],
                vocab_start: int):
        ids = ids.contiguous()
        if positions is not None:
            positions = positions.contiguous()
        out = kernels.embedding_fwd(ids, positions, tok_w, pos_w, vocab_start)
        ctx.save_for_backward(ids, positions)
        ctx.params = (tok_w, pos_w)
        ctx.vocab_start = vocab_start
        return out

    @staticmethod
    def backward(ctx, dy: Tensor):
        ids, positions = ctx.saved_tensors
        tok_w, pos_w = ctx.params
        dy = dy.contiguous()
        results = {}

        def run(tok_out, pos_out):
            kernels.embedding_bwd(ids, positions, dy, tok_out, pos_out, ctx.vocab_start)

        tok_main = getattr(tok_w, "main_grad", None)
        pos_main = getattr(pos_w, "main_grad", None) if pos_w is not None else None
        d_tok = tok_main if tok_main is not None else torch.zeros_like(tok_w)
        d_pos = None
        if pos_w is not None:
            d_pos = pos_main if pos_main is not None else torch.zeros_like(pos_w)
        run(d_tok, d_pos)
        for param, main in ((tok_w, tok_main), (pos_w, pos_main)):
            if param is not None and main is not None:
                note_grad_write(param, False)   # a scatter-add: needs what is already there
                ready = getattr(param, "_nmb_grad_ready", None)
                if ready is not None:
                    ready()
        return (None, None, None if tok_main is not None else d_tok,
                None if (pos_w is None or pos_main is not None) else d_pos, None)


def embedding(ids: Tensor, positions: Optional[Tensor], tok_w: Tensor, pos_w: Optional[Tensor],
              vocab_start: int = 0) -> Tensor:
    """``tok_w[ids - vocab_start]`` (zero rows for ids outside the shard) ``+ pos_w[positions]``."""
    if use_native(tok_w) and tok_w.shape[1] % 2 == 0:
        return _EmbeddingFn.apply(ids, positions if pos_w is not None else None, tok_w, pos_w, vocab_start)
    vloc = tok_w.shape[0]
    outside = (ids < vocab_start) | (ids >= vocab_start + vloc)
    local = (ids - vocab_start).masked_fill(outside, 0)
    out = F.embedding(local, tok_w).masked_fill(outside.unsqueeze(-1), 0.0)
    if pos_w is not None:
        out = out + F.embedding(positions, pos_w)
    return out


# ----------------------------------------------------------- cross entropy --
_CE_EXCHANGES: dict[tuple, "kernels.CeExchange"] = {}


def _ce_exchange(rows: int, device: torch.device, ws: Any) -> "kernels.CeExchange":
    """Exchange buffers per row count, kept on the workspace (tensor parallel;
    creating them is a collective over its group, like every symmetric
    allocation) or per device (single rank)."""
    cache = _CE_EXCHANGES if ws is None else ws.__dict__.setdefault("_ce_exchanges", {})
    key = (device.index, rows)
    ex = cache.get(key)
    if ex is None:
        ex = kernels.CeExchange(rows, device, ws)
        cache[key] = ex
    return ex


class _CrossEntropyFn(torch.autograd.Function):
    """Sum of token losses and number of valid tokens over vocabulary-sharded logits."""

    @staticmethod
    def forward(ctx, logits: Tensor, target: Tensor, vocab_start: int, ignore_index: int, group: Any,
                backend: Any, tp_size: int, inplace_backward: bool):
        target = target.contiguous()
        ws = None
        if tp_size > 1:
            from ..distributed import symmetric
            ws = symmetric.workspace_for(group)
        if tp_size == 1 or ws is not None:
            # ONE launch: statistics, exchange of the triples through peer memory, combine
            lse, accum = kernels.ce_forward_fused(logits, target, vocab_start, ignore_index,
                                                  _ce_exchange(logits.shape[0], logits.device, ws))
        else:
            stats = kernels.ce_stats(logits, target, vocab_start)
            gathered = torch.empty((tp_size, *stats.shape), dtype=stats.dtype, device=stats.device)
            backend.all_gather_into_tensor(gathered.view(-1, stats.shape[-1]), stats, group=group)
            lse, accum, _ = kernels.ce_combine(gathered, target, ignore_index)
        ctx.save_for_backward(logits, target, lse)
        ctx.meta = (vocab_start, ignore_index, inplace_backward)
        loss_sum, count = accum[0], accum[1]
        ctx.mark_non_differentiable(count)
        return loss_sum, count

    @staticmethod
    def backward(ctx, g_sum: Tensor, _g_count):
        logits, target, lse = ctx.saved_tensors
        vocab_start, ignore_index, inplace = ctx.meta
        gscale = g_sum.to(torch.float32).reshape(1).contiguous()
        dlogits = kernels.ce_bwd(logits, target, vocab_start, ignore_index, lse, gscale,
                                 out=logits if inplace else None)
        return dlogits, None, None, None, None, None, None, None


def cross_entropy_sum(logits2d: Tensor, target1d: Tensor, *, vocab_start: int = 0, ignore_index: int = -100,
                      group: Any = None, backend: Any = None, tp_size: int = 1,
                      inplace_backward: bool = False) -> tuple[Tensor, Tensor]:
    """Returns ``(sum of per-token losses, number of non-ignored tokens)`` as fp32 scalars.

    ``logits2d`` is ``[N, V/tp]`` (this rank's vocabulary shard starting at
    ``vocab_start``); one all-gather of three floats per token replaces the
    three all-reduces of the reference.  bf16 CUDA only.
    """
    assert use_native(logits2d)
    if logits2d.stride(-1) != 1:
        logits2d = logits2d.contiguous()
    return _CrossEntropyFn.apply(logits2d, target1d, vocab_start, ignore_index, group, backend, tp_size,
                                 inplace_backward)
