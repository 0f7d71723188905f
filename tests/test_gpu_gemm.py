"""tcgen05 GEMM against an fp32 PyTorch product of the same bf16 inputs."""
from __future__ import annotations

import pytest
import torch

from tests._numerics import assert_rel_fro

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
    assert_rel_fro(out, ref, 5e-3, "gemm")  # bf16 rounding of the output is ~2e-3


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
    assert_rel_fro(out, want, 5e-3, "bias + residual epilogue")

    aux = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    g = gemm_bf16(a, b, bias=bias, mode=EPI_GELU, aux_out=aux)
    h = ref + bias.float()
    assert (aux.float() - h).abs().max().item() < 5e-2
    assert (g.float() - torch.nn.functional.gelu(aux.float())).abs().max().item() < 2e-2
    assert_rel_fro(aux, h, 5e-3, "pre-activation")
    assert_rel_fro(g, torch.nn.functional.gelu(h), 1e-2, "GELU epilogue")

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


def _rel(got, want):
    return (got.float() - want).norm().item() / (want.norm().item() + 1e-9)


@pytest.mark.parametrize("d,hq,hkv", [(64, 4, 4), (128, 2, 1), (96, 3, 1)])
def test_rope_epilogue_and_its_undo_in_attention_backward(d, hq, hkv):
    """QKV projection whose epilogue rotates q and k (interleaved pairs, as the
    reference's apply_rotary_emb) followed by packed attention whose backward
    un-rotates dq / dk: outputs and all gradients against fp32 autograd through
    projection -> rotation -> causal attention."""
    from nano_megatron_b200.ops import functional as OF
    from nano_megatron_b200.ops.attention import flash_attention_packed
    from nano_megatron_b200.ops.gemm import RopeSpec
    from nano_megatron_b200.reference.layers import apply_rotary_emb, precompute_freqs_cis

    torch.manual_seed(5)
    b, s, h = 2, 256, 192
    n = (hq + 2 * hkv) * d
    x = _rand((b, s, h), 0.5).requires_grad_(True)
    w = _rand((n, h), 0.08).requires_grad_(True)
    bias = _rand((n,), 0.1).requires_grad_(True)
    positions = torch.arange(s, device="cuda").unsqueeze(0).expand(b, -1).contiguous()
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2, device="cuda").float() / d))
    spec = RopeSpec(RopeSpec.make_table(inv_freq, s), positions, (hq + hkv) * d)
    scale = d ** -0.5
    qkv = OF.linear(x, w, bias, rope=spec)
    out = flash_attention_packed(qkv, hq, hkv, d, scale, rope=spec)
    g = _rand(out.shape, 1.0)
    out.backward(g)

    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, bias))
    y = xf @ wf.t() + bf
    q = y[..., : hq * d].view(b, s, hq, d).transpose(1, 2)
    k = y[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d).transpose(1, 2)
    v = y[..., (hq + hkv) * d:].view(b, s, hkv, d).transpose(1, 2)
    ang = precompute_freqs_cis(d, s).to("cuda")[positions]
    q, k = apply_rotary_emb(q, ang), apply_rotary_emb(k, ang)
    # the rotated projection output itself
    want_qkv = torch.cat([q.transpose(1, 2).reshape(b, s, -1), k.transpose(1, 2).reshape(b, s, -1),
                          y[..., (hq + hkv) * d:]], dim=-1)
    assert _rel(qkv, want_qkv.detach()) < 1e-2
    rep = hq // hkv
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale).transpose(1, 2)
    assert _rel(out, ref.detach()) < 2e-2
    ref.backward(g.float())
    assert _rel(x.grad, xf.grad) < 3e-2
    assert _rel(w.grad, wf.grad) < 3e-2
    assert _rel(bias.grad, bf.grad) < 3e-2


@pytest.mark.parametrize("m,f,k,with_bias", [(512, 256, 128, True), (384, 160, 192, False), (4096, 2048, 1024, False)])
def test_swiglu_epilogues(m, f, k, with_bias):
    """fc1 with silu(gate) * up in its epilogue and fc2 whose dgrad epilogue
    applies the SwiGLU backward, against fp32 autograd."""
    from nano_megatron_b200.ops import functional as OF

    torch.manual_seed(6)
    h = 256
    x = _rand((m, k), 0.5).requires_grad_(True)
    w1 = _rand((2 * f, k), 0.1).requires_grad_(True)
    b1 = _rand((2 * f,), 0.2).requires_grad_(True) if with_bias else None
    w2 = _rand((h, f), 0.1).requires_grad_(True)
    pre, act = OF.linear_act_split(x, w1, b1, "swiglu")
    y = OF.linear_from_act(pre, act, w2, None, None, "swiglu")
    g = _rand(y.shape, 1.0)
    y.backward(g)

    xf, w1f, w2f = (t.detach().float().requires_grad_(True) for t in (x, w1, w2))
    b1f = b1.detach().float().requires_grad_(True) if with_bias else None
    pf = xf @ w1f.t() + (b1f if with_bias else 0.0)
    af = torch.nn.functional.silu(pf[:, :f]) * pf[:, f:]
    yf = af @ w2f.t()
    assert _rel(pre, pf.detach()) < 1e-2 and _rel(act, af.detach()) < 1.5e-2 and _rel(y, yf.detach()) < 2e-2
    yf.backward(g.float())
    assert _rel(x.grad, xf.grad) < 3e-2
    assert _rel(w1.grad, w1f.grad) < 3e-2 and _rel(w2.grad, w2f.grad) < 3e-2
    if with_bias:
        assert _rel(b1.grad, b1f.grad) < 3e-2


@pytest.mark.parametrize("m,n,k", [(1024, 1024, 4096), (768, 512, 2048), (3072, 1024, 4096), (256, 384, 8192)])
@pytest.mark.parametrize("accumulate", [False, True])
def test_split_k_weight_gradient(m, n, k, accumulate):
    """Weight-gradient layout (both operands MN-major) with few output tiles and a
    long K: the K range is split over CTAs, partial tiles are summed by the last
    split of a tile in split order.  Same result as fp32, bit-identical from run
    to run, and accumulation into an existing gradient works."""
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.ops.gemm import gemm_bf16

    torch.manual_seed(3)
    a, b = _rand((k, m), 0.3), _rand((k, n), 0.3)
    base = _rand((m, n), 1.0)
    ref = a.float().t() @ b.float() + (base.float() if accumulate else 0.0)
    outs = []
    native.enable_split_k(torch.cuda.current_device(), True)      # off by default
    try:
        for _ in range(3):
            out = base.clone() if accumulate else torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            gemm_bf16(a, b, a_mn=True, b_mn=True, out=out, accumulate=accumulate)
            outs.append(out)
        torch.cuda.synchronize()
    finally:
        native.enable_split_k(torch.cuda.current_device(), False)
    native.check_status()
    assert _rel(outs[0], ref) < 1e-2
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
