"""tcgen05 GEMM against an fp32 PyTorch product of the same bf16 inputs."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    A = a.float().t() if a_mn else a.float()
    B = b.float().t() if b_mn else b.float()
    return A @ B.t()


def _rand(shape, scale=1.0):
    return (torch.randn(shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 384, 192), (4096, 1024, 1024), (200, 136, 72), (384, 50304 // 8, 256)])
def test_gemm_layouts(a_mn, b_mn, m, n, k):
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.ops.gemm import gemm_bf16

    torch.manual_seed(0)
    a = _rand((k, m) if a_mn else (m, k))
    b = _rand((k, n) if b_mn else (n, k))
    out = gemm_bf16(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    native.check_status()
    ref = _ref(a, b, a_mn, b_mn)
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * ref.abs().max().item() + 1e-3
    assert err <= tol, f"max err {err} > {tol}"


def test_gemm_epilogues():
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.ops.gemm import EPI_DGELU, EPI_GELU, gemm_bf16

    torch.manual_seed(1)
    m, n, k = 512, 768, 256
    a, b = _rand((m, k), 0.5), _rand((n, k), 0.1)
    bias, res = _rand((n,)), _rand((m, n))
    ref = a.float() @ b.float().t()

    out = gemm_bf16(a, b, bias=bias, residual=res)
    want = ref + bias.float() + res.float()
    assert (out.float() - want).abs().max().item() < 5e-2

    aux = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    g = gemm_bf16(a, b, bias=bias, mode=EPI_GELU, aux_out=aux)
    h = ref + bias.float()
    assert (aux.float() - h).abs().max().item() < 5e-2
    assert (g.float() - torch.nn.functional.gelu(aux.float())).abs().max().item() < 2e-2

    dg = gemm_bf16(a, b, mode=EPI_DGELU, aux_in=aux)
    x = aux.float().requires_grad_(True)
    torch.nn.functional.gelu(x).backward(torch.ones_like(x))
    want = ref * x.grad
    assert (dg.float() - want).abs().max().item() < 5e-2 * max(1.0, want.abs().max().item())

    acc = torch.ones((m, n), dtype=torch.float32, device="cuda")
    gemm_bf16(a, b, out=acc, accumulate=True, alpha=0.5)
    assert (acc - (1.0 + 0.5 * ref)).abs().max().item() < 1e-2
    torch.cuda.synchronize()
    native.check_status()


def test_gemm_repeatable():
    from nano_megatron_b200.ops.gemm import gemm_bf16

    torch.manual_seed(2)
    a, b = _rand((1024, 512)), _rand((2048, 512))
    first = gemm_bf16(a, b)
    for _ in range(10):
        assert torch.equal(first, gemm_bf16(a, b))


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("m,n,k", [(2048, 1024, 512), (1800, 1160, 136), (4096, 4096, 1024)])
def test_gemm_cta_pair_kernel_matches_single_cta_kernel(a_mn, b_mn, m, n, k):
    """The cta_group::2 kernel (two CTAs per 256 x 256 tile) accumulates over K in
    the same order as the single-CTA kernel: identical bits, every epilogue."""
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.ops.gemm import EPI_DGELU, EPI_GELU, gemm_bf16

    torch.manual_seed(3)
    lib = native.lib()
    a = _rand((k, m) if a_mn else (m, k), 0.5)
    b = _rand((k, n) if b_mn else (n, k), 0.1)
    bias, res = _rand((n,)), _rand((m, n))
    outs = {}
    prev = lib.nmb_gemm_set_pair(0)
    try:
        for pair in (0, 1):
            lib.nmb_gemm_set_pair(pair)
            aux = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            plain = gemm_bf16(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, residual=res)
            act = gemm_bf16(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, mode=EPI_GELU, aux_out=aux)
            dact = gemm_bf16(a, b, a_mn=a_mn, b_mn=b_mn, mode=EPI_DGELU, aux_in=aux)
            acc = torch.ones((m, n), dtype=torch.bfloat16, device="cuda")
            gemm_bf16(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, accumulate=True)
            outs[pair] = (plain, act, aux, dact, acc)
    finally:
        lib.nmb_gemm_set_pair(prev)
    torch.cuda.synchronize()
    native.check_status()
    for x, y in zip(outs[0], outs[1]):
        assert torch.equal(x, y)
    ref = _ref(a, b, a_mn, b_mn) + bias.float() + res.float()
    assert (outs[1][0].float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3
