"""Multi-process tests on CPU (Gloo): N local processes stand in for N nodes.

Oracle everywhere: the single-process ``ReferenceGPT`` on the *global* batch
with the same seed.  Each launcher test starts torchrun on this file; the
worker named in the environment runs on every rank.
"""
from __future__ import annotations

import dataclasses
import os

import pytest
import torch
import torch.distributed as dist

from tests._dist_utils import launch, run_worker_if_requested

HERE = os.path.abspath(__file__)
ATOL, RTOL = 1e-5, 1e-4
MAX_WORLD = int(os.environ.get("NMB_MAX_GLOO_WORLD", "8"))


def _setup(**cfg_kw):
    import nano_megatron_b200.parallel as P
    ctx = P.initialize_parallel(P.ParallelConfig(**cfg_kw), dist_backend="gloo")
    torch.manual_seed(1234)
    return P, ctx


def _model_cfg(**kw):
    from nano_megatron_b200.reference import ReferenceGPTConfig
    base = dict(num_layers=2, hidden_size=32, num_heads=4, vocab_size=64, max_seq_len=16, attn_backend="unfused",
                use_bias=True)
    base.update(kw)
    return ReferenceGPTConfig(**base)


def _reference(cfg, ids, labels=None):
    from nano_megatron_b200.reference import ReferenceGPT, seed_all, shifted_cross_entropy
    seed_all(7)
    ref = ReferenceGPT(cfg)
    logits = ref(ids)
    loss = shifted_cross_entropy(logits, ids if labels is None else labels)
    loss.backward()
    return ref, logits.detach(), loss.detach()


def _close(a, b, what):
    assert torch.allclose(a, b, atol=ATOL, rtol=RTOL), f"{what}: max diff {(a - b).abs().max().item()}"


def _expected_shard(name, full, ctx, cfg):
    """Slice of the reference tensor (param or grad) that this TP rank owns."""
    t, r = ctx.tensor_parallel_size, ctx.tensor_parallel_rank
    if t == 1:
        return full
    from nano_megatron_b200.parallel import blockwise_column_shard, column_shard, row_shard
    leaf = name.split(".")[-1]
    d = cfg.hidden_size // cfg.num_heads
    if "qkv_proj" in name:
        kv = cfg.num_query_groups * d
        w = full if leaf == "weight" else full.unsqueeze(1)
        out = blockwise_column_shard(w, None, r, t, (cfg.hidden_size, kv, kv))[0]
        return out if leaf == "weight" else out.squeeze(1)
    if "fc1" in name and cfg.gated_linear_unit:
        f = cfg.ffn_hidden_size
        w = full if leaf == "weight" else full.unsqueeze(1)
        out = blockwise_column_shard(w, None, r, t, (f, f))[0]
        return out if leaf == "weight" else out.squeeze(1)
    if any(k in name for k in ("q_proj", "k_proj", "v_proj", "fc1", "lm_head", "tok_emb")):
        w = full if full.dim() == 2 else full.unsqueeze(1)
        out = column_shard(w, None, r, t)[0]
        return out if full.dim() == 2 else out.squeeze(1)
    if ("out_proj" in name or "fc2" in name) and leaf == "weight":
        return row_shard(full, None, r, t)[0]
    return full  # replicated: norms, row biases, pos_emb


def _check_grads(model, ref, ctx, cfg, rename=lambda n: n):
    ref_grads = {n: p.grad for n, p in ref.named_parameters()}
    for n, p in model.named_parameters():
        want = _expected_shard(rename(n), ref_grads[rename(n)], ctx, cfg)
        assert p.grad is not None, n
        _close(p.grad, want, f"grad {n}")


# ------------------------------------------------------------------ workers --
def worker_groups():
    P, ctx = _setup(tensor_parallel_size=2)
    t = torch.tensor([float(ctx.rank + 1)])
    ctx.backend.all_reduce(t, group=ctx.tensor_parallel_group)
    base = (ctx.rank // 2) * 2
    assert t.item() == (base + 1) + (base + 2)
    d = torch.tensor([float(ctx.rank + 1)])
    ctx.backend.all_reduce(d, group=ctx.data_parallel_group)
    assert d.item() == (ctx.rank % 2 + 1) + (ctx.rank % 2 + 3)
    out = torch.empty(2)
    ctx.backend.all_gather_into_tensor(out, torch.tensor([float(ctx.rank)]), group=ctx.tensor_parallel_group)
    assert out.tolist() == [float(base), float(base + 1)]
    rs = torch.empty(1)
    ctx.backend.reduce_scatter(rs, [torch.tensor([1.0]), torch.tensor([2.0])], group=ctx.tensor_parallel_group)
    assert rs.item() == (2.0 if ctx.tensor_parallel_rank == 0 else 4.0)
    for _ in range(50):                                   # async handles may be waited and dropped
        x = torch.ones(8)
        ctx.backend.all_reduce(x, group=ctx.tensor_parallel_group, async_op=True).wait()
        assert x[0].item() == 2.0
    dist.barrier()
    P.destroy_parallel()
    assert not P.is_parallel_initialized() and not dist.is_initialized()


def worker_symmetric_backend_falls_back():
    """``SymmetricBackend`` without a GPU (no workspace, CPU tensors): every method of
    the protocol gives the library's result and is counted as a library call."""
    from nano_megatron_b200.distributed import SymmetricBackend
    import nano_megatron_b200.parallel as P
    be = SymmetricBackend()
    ctx = P.initialize_parallel(P.ParallelConfig(), dist_backend="gloo", backend=be)
    assert ctx.backend is be
    n, r = ctx.world_size, ctx.rank
    x = torch.full((5,), float(r + 1))
    assert be.all_reduce(x).tolist() == [float(n * (n + 1) // 2)] * 5
    assert be.all_reduce(torch.full((2,), float(r)), op="max", async_op=True).wait() is not None
    out = torch.empty(n * 3)
    be.all_gather_into_tensor(out, torch.full((3,), float(r)))
    assert out.view(n, 3)[:, 0].tolist() == [float(i) for i in range(n)]
    lst = [torch.empty(2) for _ in range(n)]
    be.all_gather(lst, torch.full((2,), float(r)))
    assert [t[0].item() for t in lst] == [float(i) for i in range(n)]
    rs = torch.empty(4)
    be.reduce_scatter(rs, [torch.full((4,), float(i + r)) for i in range(n)])
    assert rs[0].item() == float(sum(r + i for i in range(n)))
    b = torch.full((3,), float(r))
    be.broadcast(b, n - 1)
    assert b[0].item() == n - 1
    be.barrier()
    if r == 0:
        be.send(torch.tensor([7.0]), 1)
    elif r == 1:
        assert be.recv(torch.empty(1), 0).item() == 7.0
    assert be.counts and all(k.endswith(":library") for k in be.counts), be.counts
    assert {k.split(":")[0] for k in be.counts} == {"all_reduce", "all_gather_into_tensor", "all_gather",
                                                    "reduce_scatter", "broadcast", "barrier"}
    dist.barrier()
    P.destroy_parallel()


def _tp_worker(sp: bool, **knobs):
    from nano_megatron_b200.models import build_tp_gpt_from_reference
    P, ctx = _setup(tensor_parallel_size=2, sequence_parallel=sp)
    cfg = _model_cfg(**knobs)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    ref, ref_logits, ref_loss = _reference(cfg, ids)
    model = build_tp_gpt_from_reference(ref, ctx)
    logits = model(ids)
    parts = [torch.empty_like(logits) for _ in range(2)]
    dist.all_gather(parts, logits.detach().contiguous(), group=ctx.tensor_parallel_group)
    _close(torch.cat(parts, dim=-1), ref_logits, "logits")
    loss = model.shifted_cross_entropy(logits, ids)
    _close(loss.detach(), ref_loss, "loss")
    loss.backward()
    _check_grads(model, ref, ctx, cfg)
    P.destroy_parallel()


def worker_tp2():
    _tp_worker(False)


def worker_tp2_fused_gated_gqa():
    _tp_worker(False, use_fused_qkv=True, num_query_groups=2, gated_linear_unit=True)


def worker_tp2_gpt2_tied():
    _tp_worker(False, position_embedding_type="learned_absolute", gated_linear_unit=False, tie_word_embeddings=True,
               use_fused_qkv=True)


def worker_sp2():
    _tp_worker(True)


def worker_sp2_gpt2():
    _tp_worker(True, position_embedding_type="learned_absolute", gated_linear_unit=False, use_fused_qkv=True)


def worker_sp_equals_tp_on_same_groups():
    from nano_megatron_b200.models import build_tp_gpt_from_reference
    P, ctx = _setup(tensor_parallel_size=2)
    cfg = _model_cfg()
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    ref, _, _ = _reference(cfg, ids)
    ref.zero_grad()
    tp = build_tp_gpt_from_reference(ref, ctx)
    sp = build_tp_gpt_from_reference(ref, dataclasses.replace(ctx, sequence_parallel=True))
    a, b = tp(ids), sp(ids)
    _close(a.detach(), b.detach(), "sp vs tp logits")
    la, lb = tp.shifted_cross_entropy(a, ids), sp.shifted_cross_entropy(b, ids)
    la.backward()
    lb.backward()
    for (n, p), (_, q) in zip(tp.named_parameters(), sp.named_parameters()):
        _close(p.grad, q.grad, f"sp vs tp grad {n}")
    P.destroy_parallel()


def worker_ddp_mlp():
    from nano_megatron_b200.distributed import DistributedDataParallel
    P, ctx = _setup()
    world = ctx.world_size
    torch.manual_seed(5)
    net = torch.nn.Sequential(torch.nn.Linear(6, 16), torch.nn.Tanh(), torch.nn.Linear(16, 3))
    full = torch.nn.Sequential(torch.nn.Linear(6, 16), torch.nn.Tanh(), torch.nn.Linear(16, 3))
    full.load_state_dict(net.state_dict())
    with torch.no_grad():                                  # ranks start different; DDP must fix that
        for p in net.parameters():
            p.add_(float(ctx.rank))
    x = torch.randn(4 * world, 6)
    ddp = DistributedDataParallel(net, ctx, bucket_cap_mb=1e-4)
    for p, q in zip(net.parameters(), full.parameters()):
        assert torch.equal(p, q)
    mine = x[ctx.rank * 4:(ctx.rank + 1) * 4]
    ddp(mine).pow(2).mean().backward()
    ddp.finish_grad_sync()
    full(x).pow(2).mean().backward()
    for p, q in zip(net.parameters(), full.parameters()):
        _close(p.grad, q.grad, "ddp grad")
    ddp.zero_grad()
    with ddp.no_sync():
        ddp(mine[:2]).pow(2).mean().backward()
    ddp(mine[2:]).pow(2).mean().backward()                # accumulate, then one sync
    ddp.finish_grad_sync()
    full.zero_grad()
    sum(full(x[r * 4 + o:r * 4 + o + 2]).pow(2).mean() for r in range(world) for o in (0, 2)).div(world).backward()
    for p, q in zip(net.parameters(), full.parameters()):
        _close(p.grad, q.grad, "ddp accumulated grad")
    P.destroy_parallel()


def worker_ddp_persistent_mlp():
    from nano_megatron_b200.distributed import DistributedDataParallel
    P, ctx = _setup()
    torch.manual_seed(5)
    net = torch.nn.Sequential(torch.nn.Linear(6, 16), torch.nn.Tanh(), torch.nn.Linear(16, 3))
    full = torch.nn.Sequential(torch.nn.Linear(6, 16), torch.nn.Tanh(), torch.nn.Linear(16, 3))
    full.load_state_dict(net.state_dict())
    ddp = DistributedDataParallel(net, ctx, bucket_cap_mb=1e-4, persistent_grads=True)
    x = torch.randn(4 * ctx.world_size, 6)
    for step in range(2):
        ddp.zero_grad()
        full.zero_grad()
        ddp(x[ctx.rank * 4:(ctx.rank + 1) * 4]).pow(2).mean().backward()
        ddp.finish_grad_sync()
        full(x).pow(2).mean().backward()
        for p, q in zip(net.parameters(), full.parameters()):
            assert p.grad.data_ptr() == p.main_grad.data_ptr()
            _close(p.grad, q.grad, f"persistent ddp grad step {step}")
    P.destroy_parallel()


def worker_tp2_dp2():
    from nano_megatron_b200.distributed import DistributedDataParallel
    from nano_megatron_b200.models import build_tp_gpt_from_reference
    P, ctx = _setup(tensor_parallel_size=2)
    cfg = _model_cfg()
    ids = torch.randint(0, cfg.vocab_size, (4, 16))
    ref, _, ref_loss = _reference(cfg, ids)
    model = build_tp_gpt_from_reference(ref, ctx)
    ddp = DistributedDataParallel(model, ctx)
    mine = ids[ctx.data_parallel_rank * 2:(ctx.data_parallel_rank + 1) * 2]
    loss = model.shifted_cross_entropy(ddp(mine), mine)
    loss.backward()
    ddp.finish_grad_sync()
    _check_grads(model, ref, ctx, cfg)
    P.destroy_parallel()


def _pp_worker(tp=1, pp=2, microbatches=2, use_ddp=False, sp=False):
    from nano_megatron_b200.distributed import DistributedDataParallel
    from nano_megatron_b200.models import build_pipeline_stage_from_reference
    from nano_megatron_b200.schedules import forward_backward_1f1b
    P, ctx = _setup(tensor_parallel_size=tp, pipeline_parallel_size=pp, sequence_parallel=sp)
    cfg = _model_cfg(num_layers=4)
    dp = ctx.data_parallel_size
    ids = torch.randint(0, cfg.vocab_size, (4 * dp, 16))
    ref, _, ref_loss = _reference(cfg, ids)
    stage = build_pipeline_stage_from_reference(ref, ctx)
    ddp = DistributedDataParallel(stage, ctx) if (use_ddp or dp > 1) else None
    mine = ids[ctx.data_parallel_rank * 4:(ctx.data_parallel_rank + 1) * 4]
    loss = forward_backward_1f1b(stage=stage, ctx=ctx, input_ids=mine, labels=mine, num_microbatches=microbatches,
                                 ddp=ddp)
    if P.is_pipeline_last_stage(ctx):
        avg = loss.detach().clone()
        if dp > 1:
            dist.all_reduce(avg, group=ctx.data_parallel_group)
            avg /= dp
        _close(avg, ref_loss, "1f1b loss")
    else:
        assert loss is None
    per = cfg.num_layers // pp
    offset = ctx.pipeline_parallel_rank * per

    def rename(n):
        if n.startswith("blocks."):
            _, idx, rest = n.split(".", 2)
            return f"blocks.{int(idx) + offset}.{rest}"
        return n

    _check_grads(stage, ref, ctx, cfg, rename)
    P.destroy_parallel()


def _trainer_worker(tp=1, sp=False, cp=1):
    """``Trainer.step`` (zero-grad, forward, loss, backward, gradient sync, AdamW) for two
    steps on a sharded model against the oracle's train step on the whole model and the
    whole batch: mean loss over the data / context ranks and every parameter shard."""
    from nano_megatron_b200.engine import Trainer
    from nano_megatron_b200.models import build_tp_gpt_from_reference
    from nano_megatron_b200.reference import AdamW, shifted_cross_entropy
    P, ctx = _setup(tensor_parallel_size=tp, sequence_parallel=sp, context_parallel_size=cp)
    cfg = _model_cfg()
    dp = ctx.data_parallel_size
    ids = torch.randint(0, cfg.vocab_size, (2 * dp, 16))
    ref, _, _ = _reference(cfg, ids)
    model = build_tp_gpt_from_reference(ref, ctx)
    trainer = Trainer(model, ctx, lr=1e-2, weight_decay=0.01)
    opt = AdamW(ref.named_parameters(), lr=1e-2, weight_decay=0.01)
    mine = ids[ctx.data_parallel_rank * 2:(ctx.data_parallel_rank + 1) * 2]
    for step in range(2):
        opt.zero_grad()
        want = shifted_cross_entropy(ref(ids), ids)
        want.backward()
        opt.step()
        mean = trainer.step(mine).detach().clone()
        dist.all_reduce(mean, group=ctx.data_context_parallel_group)
        mean /= cp * dp
        _close(mean, want.detach(), f"step {step} loss")
        ref_params = dict(ref.named_parameters())
        for n, p in model.named_parameters():
            want_p = _expected_shard(n, ref_params[n].detach(), ctx, cfg)
            assert torch.allclose(p.detach(), want_p, atol=3e-4, rtol=1e-4), \
                f"step {step} {n}: max diff {(p.detach() - want_p).abs().max().item()}"
    trainer.close()
    P.destroy_parallel()


def worker_trainer_dp2():
    _trainer_worker()


def worker_trainer_tp2_sp():
    _trainer_worker(tp=2, sp=True)


def worker_trainer_tp2_dp2():
    _trainer_worker(tp=2)


def worker_trainer_cp2():
    _trainer_worker(cp=2)


def _pipeline_trainer_worker(tp=1, pp=2, microbatches=2):
    """``PipelineTrainer`` (eager 1F1B on a CPU) for two optimisation steps against the
    oracle's train step on the whole model: loss on the last stage, gradients after
    ``forward_backward`` and parameters after ``step`` on every stage."""
    from nano_megatron_b200.engine import PipelineTrainer
    from nano_megatron_b200.models import build_pipeline_stage_from_reference
    from nano_megatron_b200.reference import AdamW, shifted_cross_entropy
    P, ctx = _setup(tensor_parallel_size=tp, pipeline_parallel_size=pp)
    cfg = _model_cfg(num_layers=4)
    dp = ctx.data_parallel_size
    ids = torch.randint(0, cfg.vocab_size, (4 * dp, 16))
    ref, _, ref_loss = _reference(cfg, ids)
    stage = build_pipeline_stage_from_reference(ref, ctx)
    trainer = PipelineTrainer(stage, ctx, num_microbatches=microbatches, lr=1e-2, weight_decay=0.01)
    assert not trainer.graphed
    mine = ids[ctx.data_parallel_rank * 4:(ctx.data_parallel_rank + 1) * 4]
    per = cfg.num_layers // pp
    offset = ctx.pipeline_parallel_rank * per

    def rename(n):
        if n.startswith("blocks."):
            _, idx, rest = n.split(".", 2)
            return f"blocks.{int(idx) + offset}.{rest}"
        return n

    def check_loss(loss, want):
        if P.is_pipeline_last_stage(ctx):
            avg = loss.detach().clone()
            if dp > 1:
                dist.all_reduce(avg, group=ctx.data_parallel_group)
                avg /= dp
            _close(avg, want, "pipeline trainer loss")
        else:
            assert loss is None

    check_loss(trainer.forward_backward(mine), ref_loss)
    _check_grads(stage, ref, ctx, cfg, rename)
    opt = AdamW(ref.named_parameters(), lr=1e-2, weight_decay=0.01)
    for step in range(2):
        opt.zero_grad()
        want = shifted_cross_entropy(ref(ids), ids)
        want.backward()
        opt.step()
        check_loss(trainer.step(mine), want.detach())
        ref_params = dict(ref.named_parameters())
        for n, p in stage.named_parameters():
            # Adam turns a rounding-level difference of a gradient (the data-parallel mean is
            # summed in another order) into a visible fraction of lr = 1e-2: looser than _close
            want_p = _expected_shard(rename(n), ref_params[rename(n)].detach(), ctx, cfg)
            assert torch.allclose(p.detach(), want_p, atol=3e-4, rtol=1e-4), \
                f"step {step} {n}: max diff {(p.detach() - want_p).abs().max().item()}"
    trainer.close()
    P.destroy_parallel()


def worker_pipeline_trainer_pp2():
    _pipeline_trainer_worker()


def worker_pipeline_trainer_tp2_pp2():
    _pipeline_trainer_worker(tp=2)


def worker_pipeline_trainer_dp2_pp2():
    _pipeline_trainer_worker()          # world 4 with pp 2 leaves a data-parallel size of 2


def worker_pp2():
    _pp_worker()


def worker_pp4_m8():
    _pp_worker(pp=4, microbatches=4)


def worker_tp2_pp2():
    _pp_worker(tp=2)


def worker_tp2_pp2_sp():
    _pp_worker(tp=2, sp=True)


def worker_dp2_pp2():
    _pp_worker(use_ddp=True)


def worker_tp2_dp2_pp2():
    _pp_worker(tp=2, use_ddp=True)


def _cp_worker(tp=1):
    from nano_megatron_b200.distributed import DistributedDataParallel
    from nano_megatron_b200.models import build_tp_gpt_from_reference, tp_gpt
    P, ctx = _setup(tensor_parallel_size=tp, context_parallel_size=2)
    cfg = _model_cfg()
    dp = ctx.data_parallel_size
    ids = torch.randint(0, cfg.vocab_size, (2 * dp, 16))
    labels = ids.clone()
    labels[0, 4] = -100
    ref, ref_logits, ref_loss = _reference(cfg, ids, labels)
    model = build_tp_gpt_from_reference(ref, ctx)
    ddp = DistributedDataParallel(model, ctx)
    sl = slice(ctx.data_parallel_rank * 2, (ctx.data_parallel_rank + 1) * 2)
    logits = ddp(ids[sl])
    assert logits.shape[1] == 8                            # local sequence shard
    # reassemble over vocab (TP) then sequence (CP) for the comparison only
    v_parts = [torch.empty_like(logits) for _ in range(tp)]
    dist.all_gather(v_parts, logits.detach().contiguous(), group=ctx.tensor_parallel_group)
    local_full_v = torch.cat(v_parts, dim=-1)
    s_parts = [torch.empty_like(local_full_v) for _ in range(2)]
    dist.all_gather(s_parts, local_full_v, group=ctx.context_parallel_group)
    _close(torch.cat(s_parts, dim=1), ref_logits[sl], "cp logits")

    def no_gather(*a, **k):                                # the loss must stay local
        raise AssertionError("CE gathered logits over the CP group")

    saved = tp_gpt.gather_from_context_parallel_region
    tp_gpt.gather_from_context_parallel_region = no_gather
    try:
        loss = model.shifted_cross_entropy(logits, labels[sl])
    finally:
        tp_gpt.gather_from_context_parallel_region = saved
    mean = loss.detach().clone()
    dist.all_reduce(mean, group=ctx.data_context_parallel_group)
    mean /= (2 * dp)
    if dp == 1:
        _close(mean, ref_loss, "cp mean loss")
    loss.backward()
    ddp.finish_grad_sync()
    if dp == 1:
        _check_grads(model, ref, ctx, cfg)
    else:
        # DDP mean over DPxCP of per-DP-rank full-sequence means == global mean
        # only when every DP shard has the same number of valid tokens.
        from nano_megatron_b200.reference import ReferenceGPT, seed_all, shifted_cross_entropy
        seed_all(7)
        ref2 = ReferenceGPT(cfg)
        sum(shifted_cross_entropy(ref2(ids[r * 2:(r + 1) * 2]), labels[r * 2:(r + 1) * 2]) for r in range(dp)).div(dp).backward()
        _check_grads(model, ref2, ctx, cfg)
    P.destroy_parallel()


def worker_cp2():
    _cp_worker()


def worker_cp2_tp2():
    _cp_worker(tp=2)


def worker_cp2_dp2():
    _cp_worker()


# ---------------------------------------------------------------- launchers --
CASES = [
    ("worker_groups", 4), ("worker_symmetric_backend_falls_back", 2), ("worker_tp2", 2), ("worker_tp2_fused_gated_gqa", 2), ("worker_tp2_gpt2_tied", 2),
    ("worker_sp2", 2), ("worker_sp2_gpt2", 2), ("worker_sp_equals_tp_on_same_groups", 2),
    ("worker_ddp_mlp", 2), ("worker_ddp_mlp", 4), ("worker_ddp_persistent_mlp", 2), ("worker_tp2_dp2", 4),
    ("worker_trainer_dp2", 2), ("worker_trainer_tp2_sp", 2), ("worker_trainer_tp2_dp2", 4), ("worker_trainer_cp2", 2),
    ("worker_pipeline_trainer_pp2", 2), ("worker_pipeline_trainer_tp2_pp2", 4), ("worker_pipeline_trainer_dp2_pp2", 4),
    ("worker_pp2", 2), ("worker_pp4_m8", 4), ("worker_tp2_pp2", 4), ("worker_tp2_pp2_sp", 4),
    ("worker_dp2_pp2", 4), ("worker_tp2_dp2_pp2", 8), ("worker_cp2", 2), ("worker_cp2_tp2", 4),
    ("worker_cp2_dp2", 4),
]


@pytest.mark.parametrize("worker,world", CASES, ids=[f"{w}-{n}" for w, n in CASES])
def test_gloo(worker, world):
    if world > MAX_WORLD:
        pytest.skip(f"world {world} > NMB_MAX_GLOO_WORLD")
    launch(HERE, worker, world, timeout=180)


if __name__ == "__main__":
    run_worker_if_requested(globals())
