"""``Trainer.step`` on one GPU against the same step written out by hand.

Kept in a file of its own that sorts after the other GPU tests: it is the newest of them."""
from __future__ import annotations

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
        assert abs(got - loss.item()) <= 1e-2 * abs(loss.item()), (step, got, loss.item())
    torch.cuda.synchronize()
    native.check_status()
    assert trainer.graphed, trainer.graph_error
    plan = trainer.ddp._zero_plan
    assert plan is not None and len(plan[1]) > 0           # some parameters are no longer zeroed
    # Element-wise bounds are no use here: Adam's update is +-lr whatever the size of the
    # gradient, and the bf16 atomics of the embedding backward sum in a different order from
    # run to run, so single elements with a near-zero gradient may move the other way.
    from tests._numerics import rel_fro
    # Matrices only: a vector whose true gradient is zero (a key bias) walks randomly.
    worst = max(rel_fro(p, q) for p, q in zip(model.parameters(), twin.parameters()) if p.dim() > 1)
    assert worst < 2e-2, worst
