"""tcgen05 flash attention against an fp32 unfused PyTorch reference."""
from __future__ import annotations

import math

import pytest
import torch

from tests._numerics import assert_rel_fro

pytestmark = pytest.mark.gpu


def _ref(q, k, v, scale, q_pos0=0):
    # q [B,Sq,Hq,d], k/v [B,Skv,Hkv,d] -> fp32 reference with GQA repeat
    b, sq, hq, d = q.shape
    skv, hkv = k.shape[1], k.shape[2]
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(hq // hkv, dim=1)
    s = qf @ kf.transpose(-1, -2) * scale
    qpos = torch.arange(q_pos0, q_pos0 + sq, device=q.device)[:, None]
    kpos = torch.arange(skv, device=q.device)[None, :]
    s = s.masked_fill(kpos > qpos, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return (p @ vf).transpose(1, 2)


@pytest.mark.parametrize("b,s,hq,hkv,d", [(1, 128, 1, 1, 64), (2, 256, 4, 4, 64), (1, 384, 2, 2, 128),
                                          (2, 200, 4, 2, 64), (1, 256, 2, 2, 96), (2, 1024, 4, 4, 64)])
def test_flash_fwd_bwd(b, s, hq, hkv, d):
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.ops.attention import flash_attention

    torch.manual_seed(0)
    scale = 1.0 / math.sqrt(d)
    # packed [B, S, (hq + 2 hkv) * d] as a fused QKV projection would emit
    width = (hq + 2 * hkv) * d
    qkv = torch.randn(b, s, width, device="cuda").to(torch.bfloat16).requires_grad_(True)
    q = qkv[..., : hq * d].view(b, s, hq, d)
    k = qkv[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
    v = qkv[..., (hq + hkv) * d:].view(b, s, hkv, d)
    out = flash_attention(q, k, v, scale)
    torch.cuda.synchronize()
    native.check_status()
    ref_in = qkv.detach().float().requires_grad_(True)
    rq = ref_in[..., : hq * d].view(b, s, hq, d)
    rk = ref_in[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
    rv = ref_in[..., (hq + hkv) * d:].view(b, s, hkv, d)
    ref = _ref(rq, rk, rv, scale)
    assert (out.float() - ref).abs().max().item() < 2e-2
    assert_rel_fro(out, ref, 1e-2, "attention forward")
    g = torch.randn_like(ref)
    ref.backward(g)
    out.backward(g.to(torch.bfloat16))
    torch.cuda.synchronize()
    native.check_status()
    err = (qkv.grad.float() - ref_in.grad).abs().max().item()
    assert err < 5e-2 * max(1.0, ref_in.grad.abs().max().item()), err
    assert_rel_fro(qkv.grad, ref_in.grad, 2e-2, "attention backward")


@pytest.mark.parametrize("b,s,hq,hkv,d", [(2, 256, 4, 4, 64), (1, 200, 4, 2, 64), (1, 256, 2, 2, 128)])
def test_flash_packed_matches_reference_and_writes_one_gradient_buffer(b, s, hq, hkv, d):
    """The packed entry point (dQ / dK / dV written into slices of one buffer)."""
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.ops.attention import flash_attention_packed, split_packed_qkv

    torch.manual_seed(1)
    scale = 1.0 / math.sqrt(d)
    width = (hq + 2 * hkv) * d
    qkv = torch.randn(b, s, width, device="cuda").to(torch.bfloat16).requires_grad_(True)
    out = flash_attention_packed(qkv, hq, hkv, d, scale)
    ref_in = qkv.detach().float().requires_grad_(True)
    rq = ref_in[..., : hq * d].view(b, s, hq, d)
    rk = ref_in[..., hq * d: (hq + hkv) * d].view(b, s, hkv, d)
    rv = ref_in[..., (hq + hkv) * d:].view(b, s, hkv, d)
    ref = _ref(rq, rk, rv, scale)
    assert (out.float() - ref).abs().max().item() < 2e-2
    g = torch.randn_like(ref)
    ref.backward(g)
    out.backward(g.to(torch.bfloat16))
    torch.cuda.synchronize()
    native.check_status()
    bound = 5e-2 * max(1.0, ref_in.grad.abs().max().item())
    assert (qkv.grad.float() - ref_in.grad).abs().max().item() < bound
    # the differentiable split (one concatenation in backward) gives the same gradient
    qkv2 = qkv.detach().clone().requires_grad_(True)
    q, k, v = split_packed_qkv(qkv2, hq, hkv, d)
    (q.float().sum() * 2 + k.float().sum() * 3 + v.float().sum() * 5).backward()
    expect = torch.cat([torch.full((hq * d,), 2.0), torch.full((hkv * d,), 3.0), torch.full((hkv * d,), 5.0)]).cuda()
    assert torch.equal(qkv2.grad.float(), expect.expand(b, s, width))


def test_flash_chunked_query_offset():
    """Simulated context-parallel rank 1 of 2: queries are the second half."""
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.ops.attention import attn_bwd, attn_fwd

    torch.manual_seed(1)
    b, s, h, d = 1, 512, 2, 64
    scale = 1.0 / math.sqrt(d)
    q = torch.randn(b, s, h, d, device="cuda").to(torch.bfloat16)
    k = torch.randn(b, s, h, d, device="cuda").to(torch.bfloat16)
    v = torch.randn(b, s, h, d, device="cuda").to(torch.bfloat16)
    half = s // 2
    kc = [k[:, :half].contiguous(), k[:, half:].contiguous()]
    vc = [v[:, :half].contiguous(), v[:, half:].contiguous()]
    q1 = q[:, half:].contiguous()
    out, lse = attn_fwd(q1, kc, vc, scale, q_pos0=half)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q1, k, v))
    ref = _ref(qf, kf, vf, scale, q_pos0=half)
    torch.cuda.synchronize()
    native.check_status()
    assert (out.float() - ref).abs().max().item() < 2e-2
    g = torch.randn_like(ref)
    ref.backward(g)
    dq, dk, dv = attn_bwd(q1, kc, vc, out, g.to(torch.bfloat16), lse, scale, q_pos0=half)
    torch.cuda.synchronize()
    native.check_status()
    assert (dq.float() - qf.grad).abs().max().item() < 5e-2
    assert (torch.cat(dk, 1).float() - kf.grad).abs().max().item() < 5e-2
    assert (torch.cat(dv, 1).float() - vf.grad).abs().max().item() < 5e-2
