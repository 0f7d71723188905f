"""Memory-bound sm_100a kernels (norm, CE, embedding, activations, RoPE,
AdamW) against fp32 PyTorch expressions of the same maths."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


@pytest.mark.parametrize("rows,h", [(64, 64), (300, 1024), (4096, 1536), (7, 130)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(rows, h, rms):
    from nano_megatron_b200.ops import functional as OF
    from nano_megatron_b200.reference.layers import rms_norm

    torch.manual_seed(0)
    x, w, b = _bf(rows, h), _bf(h) * 0.5 + 1, _bf(h)
    x.requires_grad_(True); w.requires_grad_(True); b.requires_grad_(True)
    y = OF.rms_norm(x, w, 1e-5) if rms else OF.layer_norm(x, w, b, 1e-5)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    ref = rms_norm(xf, wf, 1e-5) if rms else F.layer_norm(xf, (h,), wf, bf, 1e-5)
    assert (y.float() - ref).abs().max().item() < 4e-2
    g = _bf(rows, h)
    y.backward(g)
    ref.backward(g.float())
    assert (x.grad.float() - xf.grad).abs().max().item() < 5e-2 * max(1.0, xf.grad.abs().max().item())
    tol = 2e-2 * max(1.0, wf.grad.abs().max().item())
    assert (w.grad.float() - wf.grad).abs().max().item() < tol
    if not rms:
        assert (b.grad.float() - bf.grad).abs().max().item() < 2e-2 * max(1.0, bf.grad.abs().max().item())


@pytest.mark.parametrize("rows,h", [(512, 1024), (300, 1536)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_with_residual_folds_branch_gradient_and_accumulates_param_grads(rows, h, rms):
    """y = f(norm(x)) + x: the residual gradient is added inside the dx kernel and
    dgamma / dbeta are accumulated into the parameters' persistent buffers."""
    from nano_megatron_b200.ops import functional as OF
    from nano_megatron_b200.reference.layers import rms_norm

    torch.manual_seed(0)
    x, w, b = _bf(rows, h), _bf(h) * 0.5 + 1, _bf(h)
    x.requires_grad_(True); w.requires_grad_(True); b.requires_grad_(True)
    seed_w, seed_b = _bf(h), _bf(h)
    fired = []
    for p, seed in ((w, seed_w), (b, seed_b)):
        p.main_grad = seed.clone()
        p._nmb_grad_ready = (lambda p=p: fired.append(p))
    mult = _bf(rows, h)
    y, xr = OF.norm_with_residual(x, w, b, 1e-5, rms)
    out = y * mult + xr
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    nf = rms_norm(xf, wf, 1e-5) if rms else F.layer_norm(xf, (h,), wf, bf, 1e-5)
    ref = nf * mult.float() + xf
    g = _bf(rows, h)
    out.backward(g)
    ref.backward(g.float())
    assert (x.grad.float() - xf.grad).abs().max().item() < 5e-2 * max(1.0, xf.grad.abs().max().item())
    assert w.grad is None and fired[0] is w
    expect_w = seed_w.float() + wf.grad
    assert (w.main_grad.float() - expect_w).abs().max().item() < 3e-2 * max(1.0, expect_w.abs().max().item())
    if not rms:
        assert b.grad is None and fired[1] is b
        expect_b = seed_b.float() + bf.grad
        assert (b.main_grad.float() - expect_b).abs().max().item() < 3e-2 * max(1.0, expect_b.abs().max().item())


@pytest.mark.parametrize("rows,h,acc", [(4096, 4096, False), (1000, 1024, True), (33, 130, False), (512, 3072, True)])
def test_col_sum_single_launch_and_repeatable(rows, h, acc):
    """Bias-gradient column sum; the in-kernel finish must leave its arrival
    counters clean, so a second call gives the same answer."""
    from nano_megatron_b200.ops import kernels

    torch.manual_seed(0)
    dy = _bf(rows, h)
    ref = dy.float().sum(0)
    for _ in range(2):
        seed = _bf(h)
        out = seed.clone()
        kernels.col_sum(dy, out=out, accumulate=acc)
        expect = ref + seed.float() if acc else ref
        assert (out.float() - expect).abs().max().item() < 2e-2 * max(1.0, expect.abs().max().item())


@pytest.mark.parametrize("n,v", [(64, 128), (1000, 50304), (33, 1000)])
def test_cross_entropy_single_rank(n, v):
    from nano_megatron_b200.ops import functional as OF

    torch.manual_seed(1)
    logits = _bf(n, v, scale=2.0).requires_grad_(True)
    target = torch.randint(0, v, (n,), device=DEV)
    target[::7] = -100
    total, count = OF.cross_entropy_sum(logits, target)
    ref_in = logits.detach().float().requires_grad_(True)
    ref = F.cross_entropy(ref_in, target, ignore_index=-100, reduction="sum")
    assert count.item() == (target != -100).sum().item()
    assert abs(total.item() - ref.item()) < 2e-3 * abs(ref.item()) + 1e-3
    (total / count).backward()
    (ref / count).backward()
    assert (logits.grad.float() - ref_in.grad).abs().max().item() < 1e-3


@pytest.mark.parametrize("n,v", [(33, 1000), (130, 50304), (5, 77)])
def test_one_launch_cross_entropy_forward(n, v):
    """Statistics + combine in one launch (single pass over the logits with a
    rescaled running sum), three calls in a row on different data: the gather
    buffer alternates with the device-side epoch and nothing leaks between calls."""
    from nano_megatron_b200.ops import kernels

    torch.manual_seed(11)
    ex = kernels.CeExchange(n, torch.device(DEV))
    for trial in range(3):
        # growing maxima along the row exercise the rescaling of the running sum
        logits = (_bf(n, v, scale=4.0).float() + torch.linspace(-6, 6, v, device=DEV) * (trial - 1)).to(torch.bfloat16)
        target = torch.randint(0, v, (n,), device=DEV)
        target[::5] = -100
        lse, accum = kernels.ce_forward_fused(logits, target, 0, -100, ex)
        ref_lse = torch.logsumexp(logits.float(), -1)
        assert (lse - ref_lse).abs().max().item() < 2e-3
        ref = F.cross_entropy(logits.float(), target, ignore_index=-100, reduction="sum")
        assert abs(accum[0].item() - ref.item()) < 1e-3 * abs(ref.item()) + 1e-3
        assert accum[1].item() == (target != -100).sum().item()


def test_cross_entropy_two_simulated_vocab_shards():
    from nano_megatron_b200.ops import kernels

    torch.manual_seed(2)
    n, v = 257, 512
    logits = _bf(n, v, scale=3.0)
    target = torch.randint(0, v, (n,), device=DEV)
    halves = [logits[:, : v // 2].contiguous(), logits[:, v // 2:].contiguous()]
    stats = torch.stack([kernels.ce_stats(halves[r], target, r * v // 2) for r in range(2)])
    lse, accum, rows = kernels.ce_combine(stats, target, -100, want_rows=True)
    ref = F.cross_entropy(logits.float(), target, reduction="none")
    assert (rows - ref).abs().max().item() < 2e-3
    assert (lse - torch.logsumexp(logits.float(), -1)).abs().max().item() < 2e-3
    gs = torch.ones(1, device=DEV)
    d = torch.cat([kernels.ce_bwd(halves[r], target, r * v // 2, -100, lse, gs) for r in range(2)], dim=1)
    want = torch.softmax(logits.float(), -1) - F.one_hot(target, v).float()
    assert (d.float() - want).abs().max().item() < 8e-3


def test_embedding_fwd_bwd_with_shard_and_positions():
    from nano_megatron_b200.ops import functional as OF

    torch.manual_seed(3)
    v, h, b, s = 200, 64, 2, 50
    tok = _bf(v, h).requires_grad_(True)
    pos = _bf(s, h).requires_grad_(True)
    ids = torch.randint(0, 2 * v, (b, s), device=DEV)           # half the ids belong to "another rank"
    positions = torch.arange(s, device=DEV).unsqueeze(0).expand(b, -1).contiguous()
    out = OF.embedding(ids, positions, tok, pos, vocab_start=v)
    own = (ids >= v) & (ids < 2 * v)
    tf, pf = tok.detach().float().requires_grad_(True), pos.detach().float().requires_grad_(True)
    ref = F.embedding((ids - v).clamp(0, v - 1), tf) * own.unsqueeze(-1) + F.embedding(positions, pf)
    assert (out.float() - ref).abs().max().item() < 2e-2
    g = _bf(b, s, h)
    out.backward(g)
    ref.backward(g.float())
    assert (tok.grad.float() - tf.grad).abs().max().item() < 3e-2
    assert (pos.grad.float() - pf.grad).abs().max().item() < 3e-2


def test_activations_and_rope():
    from nano_megatron_b200.ops import functional as OF
    from nano_megatron_b200.reference import layers as L

    torch.manual_seed(4)
    x = _bf(37, 256, scale=2.0).requires_grad_(True)
    xf = x.detach().float().requires_grad_(True)
    for mine, ref in ((OF.gelu, L.gelu_erf), (OF.swiglu, L.swiglu)):
        x.grad = None; xf.grad = None
        y, r = mine(x), ref(xf)
        assert (y.float() - r).abs().max().item() < 1e-2 * max(1.0, r.abs().max().item())
        g = torch.randn_like(r)
        y.backward(g.to(torch.bfloat16)); r.backward(g)
        assert (x.grad.float() - xf.grad).abs().max().item() < 2e-2 * max(1.0, xf.grad.abs().max().item())
    b, s, h, d = 2, 40, 3, 64
    q = _bf(b, s, h, d).requires_grad_(True)
    positions = torch.arange(s, device=DEV).unsqueeze(0).expand(b, -1).contiguous()
    inv = (1.0 / (10000 ** (torch.arange(0, d, 2).float() / d))).to(DEV)
    out = OF.rope_bshd(q, positions, inv)
    freqs = L.precompute_freqs_cis(d, s).to(DEV)[positions]
    qf = q.detach().float().requires_grad_(True)
    ref = L.apply_rotary_emb(qf.transpose(1, 2), freqs).transpose(1, 2)
    assert (out.float() - ref).abs().max().item() < 3e-2
    g = torch.randn_like(ref)
    out.backward(g.to(torch.bfloat16)); ref.backward(g)
    assert (q.grad.float() - qf.grad).abs().max().item() < 3e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_adamw_matches_cpu_reference_update(dtype):
    from nano_megatron_b200.reference import AdamW

    torch.manual_seed(5)
    shapes = [(300, 70), (5000,), (64, 64), (3,)]
    gpu = [torch.nn.Parameter(torch.randn(*s, device=DEV).to(dtype)) for s in shapes]
    cpu = [torch.nn.Parameter(p.detach().cpu().clone()) for p in gpu]
    og = AdamW([(f"p{i}", p) for i, p in enumerate(gpu)], lr=1e-2, weight_decay=0.1)
    oc = AdamW([(f"p{i}", p) for i, p in enumerate(cpu)], lr=1e-2, weight_decay=0.1)
    for _ in range(3):
        for pg, pc in zip(gpu, cpu):
            g = torch.randn_like(pg)
            pg.grad = g
            pc.grad = g.cpu().clone()
        og.step(); oc.step()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    for i, (pg, pc) in enumerate(zip(gpu, cpu)):
        assert (pg.detach().cpu().float() - pc.detach().float()).abs().max().item() < tol
        assert (og.state[f"p{i}"]["exp_avg"].cpu() - oc.state[f"p{i}"]["exp_avg"]).abs().max().item() < 1e-5
        assert og.state[f"p{i}"]["step"] == 3
    sd = og.state_dict()
    assert sd["p0"]["exp_avg_sq"].dtype == torch.float32 and sd["p0"]["step"] == 3


def test_linear_op_with_main_grad_accumulation():
    from nano_megatron_b200.ops import functional as OF

    torch.manual_seed(6)
    x = _bf(256, 128).requires_grad_(True)
    w = torch.nn.Parameter(_bf(384, 128, scale=0.1))
    b = torch.nn.Parameter(_bf(384))
    w.main_grad = torch.zeros_like(w); b.main_grad = torch.zeros_like(b)
    fired = []
    w._nmb_grad_ready = lambda: fired.append("w")
    for _ in range(2):
        OF.linear(x, w, b, gelu=True).sum().backward()
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    (2 * F.gelu(F.linear(xf, wf, bf)).sum()).backward()
    assert w.grad is None and fired == ["w", "w"]
    assert (w.main_grad.float() - wf.grad).abs().max().item() < 3e-2 * wf.grad.abs().max().item()
    assert (b.main_grad.float() - bf.grad).abs().max().item() < 3e-2 * bf.grad.abs().max().item()
