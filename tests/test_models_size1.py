"""Parallel models at parallel size 1 must reproduce the oracle exactly."""
from __future__ import annotations

import copy

import pytest
import torch

import nano_megatron_b200.parallel as P
from nano_megatron_b200.distributed import DistributedDataParallel
from nano_megatron_b200.models import build_pipeline_stage_from_reference, build_tp_gpt_from_reference
from nano_megatron_b200.reference import ReferenceGPT, ReferenceGPTConfig, seed_all, shifted_cross_entropy
from nano_megatron_b200.schedules import forward_backward_1f1b, warmup_microbatches
from tests._dist_utils import port_for

CONFIGS = {
    "gpt2": dict(position_embedding_type="learned_absolute", gated_linear_unit=False, use_bias=True,
                 tie_word_embeddings=True, use_fused_qkv=True),
    "rope_swiglu": dict(),
    "gqa_fused": dict(num_query_groups=2, use_fused_qkv=True, use_bias=True),
}


def _cfg(**kw):
    base = dict(num_layers=2, hidden_size=32, num_heads=4, vocab_size=64, max_seq_len=16, attn_backend="unfused")
    base.update(kw)
    return ReferenceGPTConfig(**base)


@pytest.fixture
def ctx(monkeypatch, request):
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", str(port_for(request.node.nodeid)))
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.delenv("LOCAL_RANK", raising=False)
    c = P.initialize_parallel(P.ParallelConfig(), dist_backend="gloo")
    yield c
    P.destroy_parallel()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_tp_gpt_equals_reference_at_tp1(ctx, name):
    seed_all(0)
    cfg = _cfg(**CONFIGS[name])
    ref = ReferenceGPT(cfg)
    tp = build_tp_gpt_from_reference(ref, ctx)
    ref_params, tp_params = dict(ref.named_parameters()), dict(tp.named_parameters())
    assert set(ref_params) == set(tp_params)
    for n in ref_params:
        assert torch.equal(ref_params[n], tp_params[n]), n
    assert set(ref.state_dict()) == set(tp.state_dict())
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    a, b = ref(ids), tp(ids)
    assert torch.equal(a, b)
    la, lb = shifted_cross_entropy(a, ids), tp.shifted_cross_entropy(b, ids)
    assert torch.allclose(la, lb, atol=1e-6)
    la.backward()
    lb.backward()
    for n in ref_params:
        assert torch.allclose(ref_params[n].grad, tp_params[n].grad, atol=1e-6, rtol=1e-5), n


def test_sequence_parallel_flag_is_identity_at_tp1(ctx):
    import dataclasses
    seed_all(1)
    cfg = _cfg(**CONFIGS["gpt2"])
    ref = ReferenceGPT(cfg)
    sp = build_tp_gpt_from_reference(ref, dataclasses.replace(ctx, sequence_parallel=True))
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    assert torch.allclose(sp(ids), ref(ids), atol=1e-6)


def test_cp_local_loss_pairs_average_to_full_loss(ctx):
    """Patch a live model to look like each of two CP ranks: the mean of the two
    scaled local losses equals the full-sequence CE."""
    seed_all(2)
    cfg = _cfg()
    ref = ReferenceGPT(cfg)
    model = build_tp_gpt_from_reference(ref, ctx)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    ids[0, 5] = 0
    labels = ids.clone()
    labels[1, 7] = -100
    logits = model(ids)
    full = shifted_cross_entropy(logits, labels)
    parts = []
    for r in range(2):
        model._cp_size, model._cp_rank = 2, r
        parts.append(model.shifted_cross_entropy(logits[:, r * 8:(r + 1) * 8], labels))
    model._cp_size, model._cp_rank = 1, 0
    assert torch.allclose((parts[0] + parts[1]) / 2, full, atol=1e-6)
    model._cp_size = 2
    with pytest.raises(ValueError, match="full sequence"):
        model.shifted_cross_entropy(logits[:, :8], labels[:, :8])
    with pytest.raises(ValueError, match="divisible"):
        model(ids[:, :15])


def test_tp_constraints_are_validated(ctx):
    import dataclasses
    ref = ReferenceGPT(_cfg(num_heads=4))
    bad = dataclasses.replace(ctx, tensor_parallel_size=3)
    with pytest.raises(ValueError, match="not divisible"):
        build_tp_gpt_from_reference(ref, bad)


def test_pipeline_stage_pp1_is_the_full_model(ctx):
    seed_all(3)
    cfg = _cfg(**CONFIGS["gpt2"])
    ref = ReferenceGPT(cfg)
    stage = build_pipeline_stage_from_reference(ref, ctx)
    assert stage.is_first_stage and stage.is_last_stage
    assert set(dict(stage.named_parameters())) == set(dict(ref.named_parameters()))
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    assert torch.equal(stage(ids), ref(ids))
    assert torch.allclose(stage.shifted_cross_entropy(stage(ids), ids), shifted_cross_entropy(ref(ids), ids))
    with pytest.raises(ValueError):
        stage(torch.zeros(2, 16, 3))
    import dataclasses
    two = dataclasses.replace(ctx, pipeline_parallel_size=2)
    with pytest.raises(ValueError, match="tie_word_embeddings"):
        build_pipeline_stage_from_reference(ref, two)
    untied = ReferenceGPT(_cfg(num_layers=3))
    with pytest.raises(ValueError, match="divisible"):
        build_pipeline_stage_from_reference(untied, two)
    first = build_pipeline_stage_from_reference(ReferenceGPT(_cfg()), two)
    assert first.is_first_stage and not first.is_last_stage and len(first.blocks) == 1
    assert not any(n.startswith("lm_head") or n.startswith("ln_f") for n, _ in first.named_parameters())
    with pytest.raises(RuntimeError):
        first.shifted_cross_entropy(torch.zeros(1, 2, 3), torch.zeros(1, 2, dtype=torch.long))


def test_warmup_counts():
    assert [warmup_microbatches(4, r, 8) for r in range(4)] == [3, 2, 1, 0]
    assert warmup_microbatches(4, 0, 2) == 2
    for bad in ((0, 0, 1), (2, 2, 1), (2, 0, 0)):
        with pytest.raises(ValueError):
            warmup_microbatches(*bad)


def test_1f1b_pp1_equals_full_batch(ctx):
    seed_all(4)
    cfg = _cfg()
    ref = ReferenceGPT(cfg)
    stage = build_pipeline_stage_from_reference(copy.deepcopy(ref), ctx)
    ids = torch.randint(0, cfg.vocab_size, (4, 16))
    ddp = DistributedDataParallel(stage, ctx)
    loss = forward_backward_1f1b(stage=stage, ctx=ctx, input_ids=ids, labels=ids, num_microbatches=2, ddp=ddp)
    want = shifted_cross_entropy(ref(ids), ids)
    want.backward()
    assert torch.allclose(loss, want, atol=1e-6)
    ref_grads = {n: p.grad for n, p in ref.named_parameters()}
    for n, p in stage.named_parameters():
        assert torch.allclose(p.grad, ref_grads[n], atol=1e-6, rtol=1e-5), n
    with pytest.raises(ValueError):
        forward_backward_1f1b(stage=stage, ctx=ctx, input_ids=ids, labels=ids, num_microbatches=3)
    with pytest.raises(ValueError):
        forward_backward_1f1b(stage=stage, ctx=ctx, input_ids=ids, labels=ids[:, :8], num_microbatches=2)


def test_norm_with_residual_and_packed_split_cpu_paths():
    """The fused entry points have plain-PyTorch forms on CPU with the same
    values and gradients as the unfused expressions."""
    import torch
    import torch.nn.functional as F

    from nano_megatron_b200.ops import functional as OF
    from nano_megatron_b200.ops.attention import split_packed_qkv

    torch.manual_seed(0)
    x = torch.randn(3, 5, 16, requires_grad=True)
    w, b = torch.randn(16, requires_grad=True), torch.randn(16, requires_grad=True)
    y, xr = OF.norm_with_residual(x, w, b, 1e-5, False)
    (y.sin() + xr).sum().backward()
    x2 = x.detach().clone().requires_grad_(True)
    w2, b2 = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    (F.layer_norm(x2, (16,), w2, b2, 1e-5).sin() + x2).sum().backward()
    assert torch.allclose(x.grad, x2.grad, atol=1e-6) and torch.allclose(w.grad, w2.grad, atol=1e-6)
    yr, _ = OF.norm_with_residual(x.detach(), w.detach(), None, 1e-5, True)
    from nano_megatron_b200.reference.layers import rms_norm
    assert torch.allclose(yr, rms_norm(x.detach(), w.detach(), 1e-5))

    hq, hkv, d = 4, 2, 8
    qkv = torch.randn(2, 7, (hq + 2 * hkv) * d, requires_grad=True)
    q, k, v = split_packed_qkv(qkv, hq, hkv, d)
    assert q.shape == (2, 7, hq, d) and k.shape == (2, 7, hkv, d) and v.shape == (2, 7, hkv, d)
    (q.sum() * 2 + k.sum() * 3 + v.sum() * 5).backward()
    expect = torch.cat([torch.full((hq * d,), 2.0), torch.full((hkv * d,), 3.0), torch.full((hkv * d,), 5.0)])
    assert torch.equal(qkv.grad, expect.expand(2, 7, -1))


def test_destroy_parallel_without_symmetric_workspaces_is_a_noop():
    from nano_megatron_b200.distributed import symmetric

    symmetric.close_all()
    assert symmetric.workspace_for(object()) is None


@pytest.mark.parametrize("name", ["gpt2", "rope_swiglu"])
def test_trainer_on_cpu_follows_the_oracle_trajectory(ctx, name):
    """``Trainer.step`` (zero-grad, forward, CE, backward, gradient sync, AdamW)
    is the oracle's ``reference_train_step`` when nothing is parallel."""
    from nano_megatron_b200.engine import Trainer
    from nano_megatron_b200.reference import AdamW, reference_train_step

    seed_all(0)
    cfg = _cfg(**CONFIGS[name])
    ref = ReferenceGPT(cfg)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    trainer = Trainer(build_tp_gpt_from_reference(ref, ctx), ctx, lr=1e-2, weight_decay=0.01)
    assert not trainer.graphed                               # no CUDA device: eager
    opt = AdamW(ref.named_parameters(), lr=1e-2, weight_decay=0.01)
    mine = [trainer.step(ids).item() for _ in range(3)]
    want = [reference_train_step(ref, opt, ids, capture_level="minimal", step=i).loss.item() for i in range(3)]
    assert mine == pytest.approx(want, rel=1e-6, abs=1e-6)
    assert mine[2] < mine[0]
    trainer.check()
    assert trainer.graph_settled(True) and trainer.graph_settled(False)      # nothing left to capture on a CPU
    trainer.close()                                                          # detaches hooks, drops graphs
    assert not hasattr(next(trainer.model.parameters()), "_nmb_grad_ready")
