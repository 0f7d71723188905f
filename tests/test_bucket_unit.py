"""Gradient buckets in isolation (CPU, fake collectives): construction rules,
readiness bookkeeping, the three flavours of ``sync`` and its error paths."""
from __future__ import annotations

import pytest
import torch
import torch.nn as nn

from nano_megatron_b200.distributed.bucket import GradBucket, build_buckets


class _SumOfTwo:
    """Pretends a second rank holds the same gradient: all-reduce doubles."""

    def __init__(self):
        self.seen = []

    def all_reduce(self, tensor, *, group=None, op="sum", async_op=False):
        self.seen.append((tuple(tensor.shape), op, tensor.is_contiguous()))
        tensor.mul_(2)
        return tensor


def _params(*shapes, dtype=torch.float32):
    return [nn.Parameter(torch.zeros(s, dtype=dtype)) for s in shapes]


def _with_grads(ps, value=1.0):
    for i, p in enumerate(ps):
        p.grad = torch.full_like(p, value * (i + 1))
    return ps


# ---------------------------------------------------------------- building --
def test_empty_bucket_is_rejected_and_bad_cap_raises():
    with pytest.raises(ValueError):
        GradBucket([])
    with pytest.raises(ValueError):
        build_buckets(nn.Linear(2, 2), bucket_cap_mb=0)


def test_buckets_follow_reverse_registration_order():
    net = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 2))
    (bucket,) = build_buckets(net, bucket_cap_mb=1.0)
    want = [p for p in net.parameters()][::-1]
    assert [id(p) for p in bucket.params] == [id(p) for p in want]


def test_cap_starts_a_new_bucket_but_never_splits_a_parameter():
    net = nn.Sequential(nn.Linear(64, 64, bias=False), nn.Linear(64, 64, bias=False), nn.Linear(64, 64, bias=False))
    one = 64 * 64 * 4 / (1024 * 1024)
    assert [len(b.params) for b in build_buckets(net, bucket_cap_mb=2.5 * one)] == [2, 1]
    assert [len(b.params) for b in build_buckets(net, bucket_cap_mb=0.5 * one)] == [1, 1, 1]   # oversize params stay whole


def test_a_dtype_change_closes_the_bucket_and_frozen_params_are_left_out():
    net = nn.Module()
    net.a = nn.Parameter(torch.zeros(3))
    net.b = nn.Parameter(torch.zeros(3, dtype=torch.bfloat16))
    net.c = nn.Parameter(torch.zeros(3, dtype=torch.bfloat16))
    net.frozen = nn.Parameter(torch.zeros(3), requires_grad=False)
    buckets = build_buckets(net)
    assert [[p.dtype for p in b.params] for b in buckets] == [[torch.bfloat16, torch.bfloat16], [torch.float32]]
    assert all(id(net.frozen) not in {id(p) for p in b.params} for b in buckets)
    assert build_buckets(nn.Sequential()) == []


# --------------------------------------------------------------- readiness --
def test_mark_ready_reports_the_last_parameter_once():
    a, b = _params((2,), (3,))
    bucket = GradBucket([a, b])
    assert bucket.mark_ready(a) is False and bucket.has_pending_ready
    assert bucket.mark_ready(a) is False                     # duplicates do not count
    assert bucket.mark_ready(b) is True
    with pytest.raises(KeyError):
        bucket.mark_ready(nn.Parameter(torch.zeros(1)))
    bucket.reset()
    assert not bucket.has_pending_ready and not bucket.coalesced


# -------------------------------------------------------------------- sync --
def test_sync_averages_and_writes_back_every_gradient():
    ps = _with_grads(_params((2, 2), (3,)))
    bucket, be = GradBucket(ps), _SumOfTwo()
    bucket.sync(be, None, 2)
    assert bucket.coalesced and len(be.seen) == 1 and be.seen[0][0] == (7,)
    assert torch.equal(ps[0].grad, torch.full((2, 2), 1.0)) and torch.equal(ps[1].grad, torch.full((3,), 2.0))
    bucket.sync(be, None, 2)                                 # second call is a no-op until reset
    assert len(be.seen) == 1


def test_group_of_one_never_communicates_whatever_the_divisor():
    ps = _with_grads(_params((2,)))
    for dp_size, group_size in ((1, None), (4, 1)):
        bucket, be = GradBucket(ps), _SumOfTwo()
        bucket.sync(be, None, dp_size, group_size=group_size)
        assert be.seen == [] and bucket.coalesced and torch.equal(ps[0].grad, torch.ones(2))


def test_pure_context_parallel_group_reduces_with_divisor_one():
    ps = _with_grads(_params((2,)))
    bucket, be = GradBucket(ps), _SumOfTwo()
    bucket.sync(be, None, 1, group_size=2)                  # dp = 1, cp = 2: sum, no mean
    assert len(be.seen) == 1 and torch.equal(ps[0].grad, torch.full((2,), 2.0))


def test_sync_errors():
    a, b = _params((2,), (2,))
    a.grad = torch.ones(2)
    with pytest.raises(RuntimeError, match="grad=None"):
        GradBucket([a, b]).sync(_SumOfTwo(), None, 2)
    _with_grads([a, b])
    for dp_size, group_size in ((0, None), (2, 0)):
        with pytest.raises(ValueError):
            GradBucket([a, b]).sync(_SumOfTwo(), None, dp_size, group_size=group_size)


def test_non_contiguous_gradients_are_flattened_and_restored():
    p = nn.Parameter(torch.zeros(3, 4))
    p.grad = torch.arange(12.0).reshape(4, 3).t()            # a transposed view
    assert not p.grad.is_contiguous()
    want = p.grad.clone()
    bucket, be = GradBucket([p]), _SumOfTwo()
    bucket.sync(be, None, 2)
    assert be.seen[0][2] is True                             # what reaches the collective is contiguous
    assert torch.equal(p.grad, want)


# -------------------------------------------------------------- persistent --
def test_persistent_buffer_makes_gradients_views_and_folds_strays_back():
    a, b = _params((2,), (3,))
    bucket = GradBucket([a, b])
    with pytest.raises(ValueError):
        bucket.bind_persistent(torch.zeros(4))
    flat = torch.zeros(5)
    a.grad = torch.full((2,), 7.0)                           # an existing gradient is carried over
    bucket.bind_persistent(flat)
    assert a.grad.data_ptr() == flat.data_ptr() and a.main_grad is a.grad and torch.equal(flat[:2], torch.full((2,), 7.0))
    b.grad = None                                            # a caller dropped it; autograd would allocate a fresh one
    b.grad = torch.ones(3)
    calls = []
    bucket.fused_reduce = lambda buf, divisor: calls.append((buf.data_ptr(), divisor)) or True
    bucket.sync(_SumOfTwo(), None, 2)
    assert calls == [(flat.data_ptr(), 2)]                   # the device reducer got the buffer itself
    assert b.grad.data_ptr() == flat[2:].data_ptr() and torch.equal(flat[2:], torch.ones(3))
