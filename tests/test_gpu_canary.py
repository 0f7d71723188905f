"""Out-of-bounds write detection without a sanitizer: outputs are views into a
larger buffer filled with a canary value; after the kernel the canaries around
the view must be untouched.  Shapes are deliberately ragged (not multiples of
the tile sizes)."""
from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
CANARY = -12288.0  # exactly representable in bf16


def _guarded(rows: int, cols: int, dtype=torch.bfloat16, pad_rows: int = 3, pad_cols: int = 8):
    """(view [rows, cols] with row stride cols + pad_cols, whole buffer)."""
    buf = torch.full((rows + 2 * pad_rows, cols + pad_cols), CANARY, dtype=dtype, device="cuda")
    return buf[pad_rows:pad_rows + rows, :cols], buf


def _canaries_intact(buf: torch.Tensor, rows: int, cols: int, pad_rows: int = 3) -> bool:
    mask = torch.ones_like(buf, dtype=torch.bool)
    mask[pad_rows:pad_rows + rows, :cols] = False
    return bool((buf[mask].float() == CANARY).all().item())


@pytest.mark.parametrize("m,n,k", [(200, 136, 72), (1800, 1160, 136), (4096 + 40, 1024 + 24, 256)])
def test_gemm_writes_only_its_output(m, n, k):
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.ops.gemm import gemm_bf16

    torch.manual_seed(0)
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    b = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    out, buf = _guarded(m, n)
    gemm_bf16(a, b, out=out)
    torch.cuda.synchronize()
    native.check_status()
    assert _canaries_intact(buf, m, n)
    ref = a.float() @ b.float().t()
    assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3


def test_col_sum_and_norm_write_only_their_outputs():
    from nano_megatron_b200.ops import kernels, native

    torch.manual_seed(0)
    rows, h = 777, 1024
    dy = torch.randn(rows, h, device="cuda").to(torch.bfloat16)
    guard = torch.full((h + 64,), CANARY, dtype=torch.bfloat16, device="cuda")
    out = guard[32:32 + h]
    kernels.col_sum(dy, out=out)
    x = torch.randn(rows, h, device="cuda").to(torch.bfloat16)
    w = torch.ones(h, device="cuda", dtype=torch.bfloat16)
    y, mean, rstd = kernels.norm_fwd(x, w, None, 1e-5, True)
    dx, dw, _ = kernels.norm_bwd(dy, x, w, mean, rstd, True, want_bias=False)
    torch.cuda.synchronize()
    native.check_status()
    assert bool((guard[:32].float() == CANARY).all()) and bool((guard[32 + h:].float() == CANARY).all())
    assert (out.float() - dy.float().sum(0)).abs().max().item() < 2e-2 * dy.float().sum(0).abs().max().item()
    assert torch.isfinite(dx.float()).all() and torch.isfinite(dw.float()).all()


def test_attention_writes_only_its_gradient_slices():
    """Ragged sequence length: dQ / dK / dV land inside the packed gradient and
    nowhere else (the packed buffer is allocated by the op; here the unpacked
    entry point is given guarded views)."""
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.ops.attention import attn_bwd, attn_fwd

    torch.manual_seed(0)
    b, s, h, d = 1, 200, 2, 64
    q, k, v = (torch.randn(b, s, h, d, device="cuda").to(torch.bfloat16) for _ in range(3))
    scale = 1.0 / math.sqrt(d)
    out, lse = attn_fwd(q, [k], [v], scale)
    g = torch.randn_like(out)
    views, bufs = [], []
    for _ in range(3):
        view, buf = _guarded(b * s, h * d)
        views.append(view.unflatten(1, (h, d)).unsqueeze(0))
        bufs.append(buf)
    attn_bwd(q, [k], [v], out, g, lse, scale, dq=views[0], dk_chunks=[views[1]], dv_chunks=[views[2]])
    torch.cuda.synchronize()
    native.check_status()
    for buf in bufs:
        assert _canaries_intact(buf, b * s, h * d)
    dq_ref, dk_ref, dv_ref = attn_bwd(q, [k], [v], out, g, lse, scale)
    assert torch.equal(views[0], dq_ref) and torch.equal(views[1], dk_ref[0]) and torch.equal(views[2], dv_ref[0])
