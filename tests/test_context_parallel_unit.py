"""Context-parallel helpers: range arithmetic, the scatter / gather pair along
any sequence dimension for any rank count (simulated ranks), and their
argument checks."""
from __future__ import annotations

import pytest
import torch

import nano_megatron_b200.parallel as P

from ._thread_ranks import run_ranks


@pytest.mark.parametrize("size,seq", [(1, 7), (2, 16), (4, 16), (8, 64)])
def test_local_ranges_tile_the_sequence(size, seq):
    if seq % size:
        pytest.skip("covered by the error test")
    spans = [P.local_sequence_range(r, size, seq) for r in range(size)]
    assert spans[0][0] == 0 and spans[-1][1] == seq
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert len({hi - lo for lo, hi in spans}) == 1


def test_local_range_errors():
    for bad in ((0, 0, 8), (-1, 2, 8), (2, 2, 8), (0, 3, 8)):
        with pytest.raises(ValueError):
            P.local_sequence_range(*bad)


@pytest.mark.parametrize("c,seq_dim", [(2, 1), (4, 1), (2, 2), (3, 2)])
def test_scatter_then_gather_is_the_identity_with_matching_gradients(c, seq_dim):
    torch.manual_seed(0)
    shape = [2, 3, 4, 5]
    shape[seq_dim] = 6 * c
    full = torch.randn(shape)
    weight = torch.randn(shape)

    def rank_fn(rank, be):
        x = full.clone().requires_grad_(True)
        shard = P.scatter_to_context_parallel_region(x, None, be, rank, c, seq_dim=seq_dim)
        back = P.gather_from_context_parallel_region(shard, None, be, rank, c, seq_dim=seq_dim)
        (back * weight).sum().backward()
        return shard.detach(), back.detach(), x.grad

    width = 6
    for rank, (shard, back, grad) in enumerate(run_ranks(c, rank_fn)):
        assert torch.equal(shard, full.narrow(seq_dim, rank * width, width))
        assert torch.equal(back, full)
        # every rank used the whole gathered tensor with the same weight: my shard's
        # gradient arrives c times (reduce-scatter), the rest of x gets nothing
        want = torch.zeros_like(full)
        want.narrow(seq_dim, rank * width, width).copy_(c * weight.narrow(seq_dim, rank * width, width))
        assert torch.allclose(grad, want, atol=1e-6)


def test_argument_checks_of_the_region_operators():
    x = torch.randn(2, 9, 4)

    class _Never:
        def __getattr__(self, name):
            raise AssertionError(f"{name} must not be reached")

    with pytest.raises(ValueError, match="not divisible"):
        P.scatter_to_context_parallel_region(x, None, _Never(), 0, 2)
    with pytest.raises(ValueError, match="out of range"):
        P.scatter_to_context_parallel_region(x, None, _Never(), 0, 3, seq_dim=3)
    with pytest.raises(ValueError, match="dim >= 2"):
        P.scatter_to_context_parallel_region(torch.randn(9), None, _Never(), 0, 3, seq_dim=0)
    with pytest.raises(ValueError, match="grad_op"):
        P.gather_from_context_parallel_region(x, None, _Never(), 0, 3, grad_op="average")
    # a group of one never communicates and returns its input object
    assert P.gather_from_context_parallel_region(x, None, _Never(), 0, 1) is x or \
        P.gather_from_context_parallel_region(x, None, _Never(), 0, 1).data_ptr() == x.data_ptr()


def test_offset_causal_scores_equal_the_rows_of_the_full_matrix():
    from nano_megatron_b200.reference.layers import causal_attn_scores

    torch.manual_seed(1)
    q, k = torch.randn(1, 2, 12, 4), torch.randn(1, 2, 12, 4)
    full = causal_attn_scores(q, k, scale=0.5)
    for start in (0, 4, 8):
        part = P.causal_attn_scores_cp(q[:, :, start:start + 4], k, scale=0.5, query_start=start)
        want = full[:, :, start:start + 4]
        assert torch.equal(part < -1e30, want < -1e30)          # same mask
        assert torch.allclose(part, want, rtol=1e-5, atol=1e-6)
