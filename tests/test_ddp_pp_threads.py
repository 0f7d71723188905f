"""DistributedDataParallel and the 1F1B schedule on simulated ranks (threads),
with small hand-made modules so that every gradient can be compared with a
single-process computation.  Modules are built on the main thread (the global
random generator is shared between threads) and handed to the ranks."""
from __future__ import annotations

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from nano_megatron_b200.distributed import DistributedDataParallel
from nano_megatron_b200.schedules import forward_backward_1f1b

from ._thread_ranks import run_ranks, thread_context


def _mlp(seed: int) -> nn.Module:
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(6, 8), nn.Tanh(), nn.Linear(8, 3))


# --------------------------------------------------------------------- DDP --
@pytest.mark.parametrize("dp", [2, 3])
def test_ddp_broadcasts_rank0_parameters_and_averages_gradients(dp):
    torch.manual_seed(0)
    data = [torch.randn(4, 6) for _ in range(dp)]
    dense = _mlp(100)                                           # what rank 0 starts from
    torch.cat([dense(x) for x in data]).square().mean().backward()

    replicas = [_mlp(100 + r) for r in range(dp)]               # every rank starts from a different init

    def rank_fn(rank, be):
        ctx = thread_context(rank, be, dp=dp)
        ddp = DistributedDataParallel(replicas[rank], ctx, bucket_cap_mb=1e-4)     # tiny cap: one bucket per tensor
        start = [p.detach().clone() for p in ddp.module.parameters()]
        ddp(data[rank]).square().mean().backward()
        ddp.finish_grad_sync()
        ddp.finish_grad_sync()                                  # idempotent
        return start, [p.grad.clone() for p in ddp.module.parameters()], be.counts.get("all_reduce", 0)

    want_start = [p.detach() for p in dense.parameters()]
    want_grads = [p.grad for p in dense.parameters()]
    for start, grads, n_allreduce in run_ranks(dp, rank_fn):
        assert all(torch.equal(a, b) for a, b in zip(start, want_start))
        assert all(torch.allclose(a, b, atol=1e-6) for a, b in zip(grads, want_grads))
        assert n_allreduce >= 4 + 1                              # one per bucket (+ the leader election)


def test_ddp_no_sync_accumulates_locally_and_syncs_once():
    torch.manual_seed(1)
    x = [[torch.randn(2, 6) for _ in range(2)] for _ in range(2)]        # [rank][micro]
    dense = _mlp(7)
    sum(dense(x[r][m]).sum() for r in range(2) for m in range(2)).backward()

    replicas = [_mlp(7) for _ in range(2)]

    def rank_fn(rank, be):
        ddp = DistributedDataParallel(replicas[rank], thread_context(rank, be, dp=2))
        base = be.counts.get("all_reduce", 0)
        with ddp.no_sync():
            ddp(x[rank][0]).sum().backward()
        assert be.counts.get("all_reduce", 0) == base           # nothing was exchanged under no_sync
        ddp(x[rank][1]).sum().backward()
        ddp.finish_grad_sync()
        return [p.grad.clone() for p in ddp.module.parameters()]

    for grads in run_ranks(2, rank_fn):
        for g, p in zip(grads, dense.parameters()):
            assert torch.allclose(g, p.grad / 2, atol=1e-5)      # mean over the two ranks of the per-rank sums


# -------------------------------------------------------------------- 1F1B --
class _ToyStage(nn.Module):
    """Stage ``i`` of a ``p``-stage token model: embedding on the first stage,
    one mixing layer everywhere, vocabulary head + shifted CE on the last."""

    def __init__(self, index: int, n_stages: int, vocab: int = 11, hidden: int = 8) -> None:
        super().__init__()
        torch.manual_seed(1000 + index)
        self.config = type("Cfg", (), {"hidden_size": hidden})()
        self.is_first_stage, self.is_last_stage = index == 0, index == n_stages - 1
        self.embed = nn.Embedding(vocab, hidden) if self.is_first_stage else None
        self.mix = nn.Linear(hidden, hidden)
        self.head = nn.Linear(hidden, vocab) if self.is_last_stage else None

    def forward(self, x, *, positions=None):
        h = self.embed(x) if self.is_first_stage else x
        h = torch.tanh(self.mix(h))
        return self.head(h) if self.is_last_stage else h

    def shifted_cross_entropy(self, logits, labels, ignore_index=-100):
        return F.cross_entropy(logits[:, :-1].reshape(-1, logits.size(-1)), labels[:, 1:].reshape(-1),
                               ignore_index=ignore_index)


@pytest.mark.parametrize("pp,micro", [(2, 4), (3, 3), (3, 6), (4, 2), (4, 8)])
def test_1f1b_equals_the_unsplit_model_for_any_depth_and_microbatch_count(pp, micro):
    torch.manual_seed(2)
    ids = torch.randint(0, 11, (micro * 2, 7))
    stages = [_ToyStage(i, pp) for i in range(pp)]
    h = ids
    losses = []
    for m in range(micro):
        h = ids[m * 2:(m + 1) * 2]
        for st in stages:
            h = st(h)
        losses.append(stages[-1].shifted_cross_entropy(h, ids[m * 2:(m + 1) * 2]) / micro)
    want_loss = torch.stack(losses).sum()
    want_loss.backward()
    want = [[p.grad.clone() for p in st.parameters()] for st in stages]

    mine = [_ToyStage(i, pp) for i in range(pp)]                # same seeds as `stages`: identical weights

    def rank_fn(rank, be):
        ctx = thread_context(rank, be, pp=pp)
        stage = mine[ctx.pipeline_parallel_rank]
        loss = forward_backward_1f1b(stage=stage, ctx=ctx, input_ids=ids, labels=ids, num_microbatches=micro)
        return (None if loss is None else loss.detach()), [p.grad.clone() for p in stage.parameters()], be.counts

    results = run_ranks(pp, rank_fn)
    for rank, (loss, grads, counts) in enumerate(results):
        assert (loss is None) == (rank != pp - 1)
        if loss is not None:
            assert torch.allclose(loss, want_loss.detach(), atol=1e-6)
        assert all(torch.allclose(g, w, atol=1e-5) for g, w in zip(grads, want[rank]))
        # every microbatch crosses every stage boundary once in each direction
        sends = (micro if rank < pp - 1 else 0) + (micro if rank > 0 else 0)
        assert counts.get("send", 0) == sends and counts.get("recv", 0) == sends


def test_1f1b_with_data_parallel_replicas_syncs_once_at_the_end():
    torch.manual_seed(3)
    pp, dp, micro = 2, 2, 2
    ids = [torch.randint(0, 11, (micro * 2, 5)) for _ in range(dp)]

    per_rank = [_ToyStage(i, pp) for i in range(pp) for _ in range(dp)]   # global rank = pp_rank * dp + dp_rank

    def rank_fn(rank, be):
        ctx = thread_context(rank, be, pp=pp, dp=dp)
        stage = per_rank[ctx.pipeline_parallel_rank * dp + ctx.data_parallel_rank]
        ddp = DistributedDataParallel(stage, ctx)
        before = be.counts.get("all_reduce", 0)
        mine = ids[ctx.data_parallel_rank]
        forward_backward_1f1b(stage=stage, ctx=ctx, input_ids=mine, labels=mine, num_microbatches=micro, ddp=ddp)
        n_sync = be.counts.get("all_reduce", 0) - before
        return ctx.pipeline_parallel_rank, [p.grad.clone() for p in stage.parameters()], n_sync

    # single-process reference: mean over the two replicas of each stage's gradient
    want = []
    for r in range(dp):
        stages = [_ToyStage(i, pp) for i in range(pp)]
        total = 0
        for m in range(micro):
            h = ids[r][m * 2:(m + 1) * 2]
            for st in stages:
                h = st(h)
            total = total + stages[-1].shifted_cross_entropy(h, ids[r][m * 2:(m + 1) * 2]) / micro
        total.backward()
        want.append([[p.grad.clone() for p in st.parameters()] for st in stages])
    for stage_index, grads, n_sync in run_ranks(pp * dp, rank_fn):
        mean = [(a + b) / 2 for a, b in zip(want[0][stage_index], want[1][stage_index])]
        assert all(torch.allclose(g, w, atol=1e-5) for g, w in zip(grads, mean))
        assert n_sync == 1                                       # one bucket, reduced once after the last microbatch


# ------------------------------------------------- first write overwrites --
class _DirectLinear(torch.autograd.Function):
    """y = x W^T whose weight gradient goes straight into ``weight.main_grad``
    through the framework's delivery helper (what the GEMM backward does on a GPU)."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x)
        ctx.weight = weight
        return x @ weight.t()

    @staticmethod
    def backward(ctx, dy):
        from nano_megatron_b200.ops.functional import _deliver_grad

        (x,) = ctx.saved_tensors

        def compute(out, accumulate):
            g = dy.t() @ x
            if out is None:
                return g
            if accumulate:
                out.add_(g)
            else:
                out.copy_(g)
            return None

        return dy @ ctx.weight, _deliver_grad(ctx.weight, compute)


class _Toy(nn.Module):
    def __init__(self):
        super().__init__()
        torch.manual_seed(5)
        self.emb = nn.Embedding(11, 6)          # gradient arrives through autograd: must keep being zeroed
        self.w1 = nn.Parameter(torch.randn(8, 6) * 0.3)
        self.w2 = nn.Parameter(torch.randn(3, 8) * 0.3)

    def forward(self, ids):
        return _DirectLinear.apply(torch.tanh(_DirectLinear.apply(self.emb(ids), self.w1)), self.w2)


def test_first_gradient_write_of_a_step_overwrites_instead_of_a_memset():
    """After one traced backward pass the wrapper zeroes only the parameters whose
    gradient cannot be stored by its first writer; the others get a flag that makes
    that writer overwrite.  Gradients match plain autograd on every step, stale
    values included (the buffers are poisoned before each zero_grad)."""

    def rank_fn(rank, be):
        ctx = thread_context(rank, be, dp=1)
        toy = _Toy()
        ddp = DistributedDataParallel(toy, ctx, persistent_grads=True, overwrite_first_grad=True)
        plain = _Toy()
        out = []
        for step in range(4):
            ids = torch.randint(0, 11, (5,), generator=torch.Generator().manual_seed(step))
            for flat in ddp._flat_buffers:
                flat.fill_(123.0)                                  # whatever the last step left
            ddp.zero_grad()
            ddp(ids).square().sum().backward()
            ddp.finish_grad_sync()
            plain.zero_grad()
            plain(ids).square().sum().backward()
            out.append([(n, p.grad.clone(), q.grad.clone()) for (n, p), q in
                        zip(toy.named_parameters(), plain.parameters())])
        return out, ddp._zero_plan

    (steps, plan), = run_ranks(1, rank_fn)
    for grads in steps:
        for name, got, want in grads:
            assert torch.allclose(got, want, atol=1e-6), name
    ranges, covered = plan
    assert {tuple(p.shape) for p in covered} == {(8, 6), (3, 8)}      # the two direct weights
    assert len(ranges) == 1 and ranges[0][2] - ranges[0][1] == 11 * 6  # only the embedding is still zeroed


def test_after_bucket_sync_fires_once_per_bucket_and_only_when_the_bucket_is_reduced():
    """The hook a trainer uses to act on a bucket as soon as its gradients are final."""
    replicas = [_mlp(3) for _ in range(2)]
    data = [torch.randn(4, 6, generator=torch.Generator().manual_seed(r)) for r in range(2)]
    dense = _mlp(3)                                               # built here: threads share the global generator
    sum(dense(x).square().mean() for x in data).backward()
    want = {tuple(p.shape): p.grad / 2 for p in dense.parameters()}

    def rank_fn(rank, be):
        ddp = DistributedDataParallel(replicas[rank], thread_context(rank, be, dp=2), bucket_cap_mb=1e-4)
        seen: list[int] = []
        reduced_before_hook: list[bool] = []

        def hook(bucket):
            seen.append(id(bucket))
            reduced_before_hook.append(all(torch.allclose(p.grad, want[tuple(p.shape)], atol=1e-6)
                                           for p in bucket.params))

        ddp.after_bucket_sync = hook
        with ddp.no_sync():
            ddp(data[rank]).square().mean().backward()
        assert not seen                                           # nothing is reduced under no_sync
        ddp.zero_grad()
        ddp(data[rank]).square().mean().backward()
        ddp.finish_grad_sync()
        ddp.finish_grad_sync()
        return seen, reduced_before_hook, len(ddp._buckets)

    for seen, ok, n_buckets in run_ranks(2, rank_fn):
        assert len(seen) == n_buckets == len(set(seen)) == 4       # one call per bucket, none twice
        assert all(ok)                                             # the hook sees reduced (averaged) gradients


def test_close_detaches_the_wrapper_so_that_model_and_buffers_can_be_freed():
    """The gradient hooks live in the parameters' autograd metadata and refer back to the
    wrapper; without ``close()`` wrapper, module and parameters are never collected."""
    import gc
    import weakref

    def rank_fn(rank, be):
        module = _mlp(9)
        ddp = DistributedDataParallel(module, thread_context(rank, be, dp=1))
        refs = [weakref.ref(ddp), weakref.ref(module), weakref.ref(module[0].weight)]
        ddp(torch.randn(2, 6)).sum().backward()
        ddp.finish_grad_sync()
        ddp.close()
        assert not hasattr(module[0].weight, "_nmb_grad_ready")
        del ddp, module
        gc.collect()
        return [r() is None for r in refs]

    (freed,) = run_ranks(1, rank_fn)
    assert all(freed), freed
