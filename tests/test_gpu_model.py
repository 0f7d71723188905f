"""The bf16 GPU model (all native kernels) against the fp32 CPU oracle."""
from __future__ import annotations

import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture
def ctx(monkeypatch, request):
    import nano_megatron_b200.parallel as P
    from tests._dist_utils import port_for
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", str(port_for(request.node.nodeid)))
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.setenv("LOCAL_RANK", "0")
    c = P.initialize_parallel(P.ParallelConfig(), dist_backend="nccl")
    yield c
    P.destroy_parallel()


KNOBS = {
    "gpt2": dict(position_embedding_type="learned_absolute", gated_linear_unit=False, use_bias=True,
                 tie_word_embeddings=True, use_fused_qkv=True),
    "rope_swiglu_gqa": dict(num_query_groups=2, use_fused_qkv=True),
    "separate_qkv_rms": dict(normalization="rmsnorm", use_bias=True),
}


@pytest.mark.parametrize("name", list(KNOBS))
def test_bf16_model_tracks_fp32_oracle(ctx, name):
    from nano_megatron_b200.models import build_tp_gpt_from_reference
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.reference import ReferenceGPT, ReferenceGPTConfig, seed_all, shifted_cross_entropy

    seed_all(0)
    cfg = ReferenceGPTConfig(num_layers=2, hidden_size=256, num_heads=4, vocab_size=512, max_seq_len=256,
                             **KNOBS[name])
    ref = ReferenceGPT(cfg)
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() > 1:
                p.mul_(0.5)
    model = build_tp_gpt_from_reference(ref, ctx).to("cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, cfg.vocab_size, (2, 256))
    before = dict(native.launch_counts)
    logits = model(ids.cuda())
    loss = model.shifted_cross_entropy(logits, ids.cuda())
    loss.backward()
    torch.cuda.synchronize()
    native.check_status()
    if name == "rope_swiglu_gqa":
        # rotary embedding and SwiGLU ride in GEMM epilogues (and the attention backward's last
        # kernel): no stand-alone rotation or activation kernel ran, forward or backward
        for entry in ("nmb_rope", "nmb_swiglu_fwd", "nmb_swiglu_bwd"):
            assert native.launch_counts.get(entry, 0) == before.get(entry, 0), entry
    cfg_cpu = ReferenceGPTConfig(**{**cfg.__dict__, "attn_backend": "unfused"})
    ref.config = cfg_cpu
    for blk in ref.blocks:
        blk.attn.config = cfg_cpu
    ref_logits = ref(ids)
    ref_loss = shifted_cross_entropy(ref_logits, ids)
    ref_loss.backward()
    scale = ref_logits.abs().max().item()
    assert (logits.float().cpu() - ref_logits).abs().max().item() < 4e-2 * scale
    assert abs(loss.item() - ref_loss.item()) < 3e-2 * abs(ref_loss.item())
    ref_grads = dict(ref.named_parameters())
    worst = 0.0
    for n, p in model.named_parameters():
        if cfg.normalization == "rmsnorm" and n.endswith("_bias") and "ln" in n:
            continue
        g, r = p.grad.float().cpu(), ref_grads[n].grad
        rel = (g - r).norm().item() / (r.norm().item() + 1e-6)
        worst = max(worst, rel)
        assert rel < 8e-2, (n, rel)


def test_training_loss_decreases_and_matches_oracle_trajectory(ctx):
    from nano_megatron_b200.models import build_tp_gpt_from_reference
    from nano_megatron_b200.reference import AdamW, ReferenceGPT, gpt_preset, seed_all, shifted_cross_entropy

    seed_all(0)
    cfg = gpt_preset("small", attn_backend="auto")
    ref = ReferenceGPT(cfg)
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.02)
    model = build_tp_gpt_from_reference(ref, ctx).to("cuda", dtype=torch.bfloat16)
    opt = AdamW(model.named_parameters(), lr=1e-3, weight_decay=0.01)
    cpu_opt = AdamW(ref.named_parameters(), lr=1e-3, weight_decay=0.01)
    ids = torch.randint(0, cfg.vocab_size, (4, 256))
    gpu_losses, cpu_losses = [], []
    for _ in range(6):
        opt.zero_grad()
        loss = model.shifted_cross_entropy(model(ids.cuda()), ids.cuda())
        loss.backward()
        opt.step()
        gpu_losses.append(loss.item())
        cpu_opt.zero_grad()
        l2 = shifted_cross_entropy(ref(ids), ids)
        l2.backward()
        cpu_opt.step()
        cpu_losses.append(l2.item())
    assert gpu_losses[-1] < gpu_losses[0]
    for a, b in zip(gpu_losses, cpu_losses):
        assert abs(a - b) < 5e-2 * abs(b), (gpu_losses, cpu_losses)


def _small_model(ctx, seed=0):
    from nano_megatron_b200.models import build_tp_gpt_from_reference
    from nano_megatron_b200.reference import ReferenceGPT, gpt_preset, seed_all

    seed_all(seed)
    cfg = gpt_preset("small", attn_backend="auto")
    ref = ReferenceGPT(cfg)
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() > 1:
                p.normal_(0, 0.02)
    return cfg, build_tp_gpt_from_reference(ref, ctx).to("cuda", dtype=torch.bfloat16)


@pytest.mark.parametrize("overlap_optimizer", [False, True])
def test_trainer_step_equals_the_hand_written_loop(ctx, overlap_optimizer):
    """``Trainer.step`` (persistent gradient buffers whose first write of a step overwrites
    instead of a memset, CUDA-graph replay from the fourth step on, optionally the
    per-bucket optimizer update during backward) against zero_grad / forward / backward /
    AdamW written out by hand on a copy of the model: same losses, same parameters."""
    from nano_megatron_b200.engine import Trainer
    from nano_megatron_b200.ops import native
    from nano_megatron_b200.reference import AdamW

    cfg, model = _small_model(ctx)
    _, twin = _small_model(ctx)
    trainer = Trainer(model, ctx, lr=1e-3, weight_decay=0.01, bucket_cap_mb=0.5, overlap_optimizer=overlap_optimizer)
    opt = AdamW(twin.named_parameters(), lr=1e-3, weight_decay=0.01)
    gen = torch.Generator().manual_seed(7)
    for step in range(7):
        ids = torch.randint(0, cfg.vocab_size, (4, 256), generator=gen).cuda()
        got = trainer.step(ids).item()
        opt.zero_grad()
        loss = twin.shifted_cross_entropy(twin(ids), ids)
        loss.backward()
        opt.step()
        assert abs(got - loss.item()) <= 2e-3 * abs(loss.item()), (step, got, loss.item())
    torch.cuda.synchronize()
    native.check_status()
    assert trainer.graphed, trainer.graph_error
    plan = trainer.ddp._zero_plan
    assert plan is not None and len(plan[1]) > 0           # some parameters are no longer zeroed
    worst = 0.0
    for (n, p), q in zip(model.named_parameters(), twin.parameters()):
        err = (p.float() - q.float()).abs().max().item()
        worst = max(worst, err / (q.float().abs().max().item() + 1e-6))
    assert worst < 2e-2, worst
