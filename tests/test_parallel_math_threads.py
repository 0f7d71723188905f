"""Exact arithmetic of the tensor-, sequence- and context-parallel operators on
2, 3 and 4 simulated ranks (threads sharing an in-memory backend): every rank's
forward output and input gradient is compared with the single-device
expression the operator stands for."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

import nano_megatron_b200.parallel as P
from nano_megatron_b200.parallel import mappings as M
from nano_megatron_b200.parallel.context_parallel import _GatherFromContextParallelRegion

from ._thread_ranks import run_ranks


def _close(a, b, tol=1e-5):
    return (a - b).abs().max().item() <= tol * max(1.0, b.abs().max().item())


@pytest.mark.parametrize("t", [2, 4])
def test_column_then_row_parallel_linear_equals_two_dense_layers(t):
    torch.manual_seed(0)
    x = torch.randn(3, 5, 8)
    w1, b1 = torch.randn(16, 8), torch.randn(16)
    w2, b2 = torch.randn(8, 16), torch.randn(8)
    x_ref = x.clone().requires_grad_(True)
    want = F.linear(torch.tanh(F.linear(x_ref, w1, b1)), w2, b2)
    want.square().sum().backward()

    def rank_fn(rank, be):
        col = P.ColumnParallelLinear(w1, b1, rank, t, None, be)
        row = P.RowParallelLinear(w2, b2, rank, t, None, be)
        xi = x.clone().requires_grad_(True)
        out = row(torch.tanh(col(xi)))
        out.square().sum().backward()
        return out.detach(), xi.grad, col.weight.grad, row.weight.grad, be.counts

    for rank, (out, gx, gcol, grow, counts) in enumerate(run_ranks(t, rank_fn)):
        assert _close(out, want.detach()) and _close(gx, x_ref.grad)
        assert counts["all_reduce"] == 2                    # one in forward (row), one in backward (column)
        n1, n2 = 16 // t, 16 // t
        assert gcol.shape == (n1, 8) and grow.shape == (8, n2)


@pytest.mark.parametrize("t", [2, 4])
def test_sequence_parallel_region_ops_are_mutually_consistent(t):
    torch.manual_seed(1)
    full = torch.randn(2, 8, 3)

    def rank_fn(rank, be):
        src = full.clone().requires_grad_(True)
        shard = P.scatter_to_sequence_parallel_region(src, None, be, rank, t)
        back = P.gather_from_sequence_parallel_region(shard, None, be, rank, t)
        (back * (rank + 1)).sum().backward()
        partial = (full * (rank + 1)).clone().requires_grad_(True)
        mine = P.reduce_scatter_to_sequence_parallel_region(partial, None, be, rank, t)
        mine.sum().backward()
        return shard.detach(), back.detach(), src.grad, mine.detach(), partial.grad

    width = 8 // t
    total = sum(r + 1 for r in range(t))
    for rank, (shard, back, gsrc, mine, gpartial) in enumerate(run_ranks(t, rank_fn)):
        sl = slice(rank * width, (rank + 1) * width)
        assert torch.equal(shard, full[:, sl]) and torch.equal(back, full)
        # gather's backward reduce-scatters the ranks' gradients; scatter's backward gathers them
        assert torch.equal(gsrc, torch.full_like(full, float(total)))
        assert _close(mine, full[:, sl] * total)
        assert torch.equal(gpartial, torch.ones_like(full))


@pytest.mark.parametrize("c", [2, 3])
def test_context_parallel_gather_backward_modes(c):
    torch.manual_seed(2)
    s_loc = 4
    shards = [torch.randn(1, s_loc, 2) for _ in range(c)]
    weight = torch.arange(float(c * s_loc)).view(1, c * s_loc, 1)

    def rank_fn(rank, be):
        a = shards[rank].clone().requires_grad_(True)
        full = P.gather_from_context_parallel_region(a, None, be, rank, c)             # reduce-scatter backward
        (full * weight * (rank + 1)).sum().backward()
        b = shards[rank].clone().requires_grad_(True)
        full2 = _GatherFromContextParallelRegion.apply(b, None, be, rank, c, 1, "split")
        (full2 * weight).sum().backward()
        return full.detach(), a.grad, b.grad, be.counts

    want_full = torch.cat(shards, dim=1)
    total = sum(r + 1 for r in range(c))
    for rank, (full, ga, gb, counts) in enumerate(run_ranks(c, rank_fn)):
        sl = slice(rank * s_loc, (rank + 1) * s_loc)
        assert torch.equal(full, want_full)
        assert _close(ga, (weight[:, sl] * total).expand(1, s_loc, 2))   # every rank's use of my shard, summed
        assert _close(gb, weight[:, sl].expand(1, s_loc, 2))             # identical consumers: just my slice
        assert counts["all_gather_into_tensor"] == 2 and counts["reduce_scatter"] == 1


@pytest.mark.parametrize("t", [2, 4])
def test_vocab_parallel_embedding_and_cross_entropy_match_dense(t):
    torch.manual_seed(3)
    vocab, hidden, n = 16, 6, 10
    table = torch.randn(vocab, hidden)
    ids = torch.randint(0, vocab, (2, 5))
    logits = torch.randn(2, 5, vocab)
    target = torch.randint(0, vocab, (2, 5))
    target[0, 0] = -100
    dense = logits.clone().requires_grad_(True)
    want_loss = F.cross_entropy(dense.view(-1, vocab), target.view(-1), ignore_index=-100)   # mean over kept tokens
    want_loss.backward()

    def rank_fn(rank, be):
        emb = P.VocabParallelEmbedding(vocab, hidden, tp_rank=rank, tp_size=t, group=None, backend=be, weight=table)
        looked_up = emb(ids)
        lo, hi = P.vocab_range_from_global(rank, t, vocab)
        local = logits[..., lo:hi].clone().requires_grad_(True)
        loss = P.vocab_parallel_cross_entropy_from_shifted(local, target, vocab_start_index=lo, vocab_end_index=hi,
                                                           group=None, backend=be)
        shifted = P.vocab_parallel_cross_entropy(local.detach(), target, vocab_start_index=lo, vocab_end_index=hi,
                                                 group=None, backend=be)
        assert _close(shifted, F.cross_entropy(logits[:, :-1].reshape(-1, vocab), target[:, 1:].reshape(-1),
                                               ignore_index=-100))
        loss.backward()
        return looked_up.detach(), loss.detach(), local.grad, (lo, hi)

    for looked_up, loss, glocal, (lo, hi) in run_ranks(t, rank_fn):
        assert _close(looked_up, table[ids])
        assert _close(loss, want_loss.detach())
        assert _close(glocal, dense.grad[..., lo:hi])


def test_sp_replicated_parameter_gradients_are_summed_over_ranks_once():
    def rank_fn(rank, be):
        p = torch.nn.Parameter(torch.ones(3))
        q = torch.nn.Parameter(torch.ones(2))
        M.register_sequence_parallel_grad_allreduce(p, None, be)
        M.register_sequence_parallel_grad_allreduce(q, None, be)
        ((p * (rank + 1)).sum() + (q * 10 * (rank + 1)).sum()).backward()
        return p.grad.clone(), q.grad.clone(), be.counts.get("all_reduce", 0)

    for gp, gq, n_collectives in run_ranks(3, rank_fn):
        assert torch.equal(gp, torch.full((3,), 6.0)) and torch.equal(gq, torch.full((2,), 60.0))
        assert n_collectives == 1                            # both parameters in one coalesced reduction
