"""Details of the tensor-parallel building blocks on one process: what the
conjugate operators touch and leave alone, the communication-buffer cache, the
shard helpers' error paths, layer attributes, and the layout rules of
``ParallelConfig`` / ``RankGenerator``."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

import nano_megatron_b200.parallel as P
from nano_megatron_b200.parallel import mappings as M

from ._thread_ranks import run_ranks


class _Doubling:
    """all_reduce that behaves like two ranks holding the same tensor."""

    def __init__(self, lazy: bool = False):
        self.lazy, self.pending = lazy, []

    def all_reduce(self, tensor, *, group=None, op="sum", async_op=False):
        if self.lazy and async_op:
            backend = self

            class _Work:
                def wait(self_inner):
                    tensor.mul_(2)
                    backend.pending.remove(self_inner)

            work = _Work()
            self.pending.append(work)
            return work
        tensor.mul_(2)
        return tensor


# ------------------------------------------------- conjugate operator pair --
def test_copy_to_region_is_identity_forward_and_leaves_its_input_alone():
    x = torch.arange(6.0).view(2, 3).requires_grad_(True)
    before = x.detach().clone()
    y = M._CopyToTPRegion.apply(x, None, _Doubling(), None)
    assert torch.equal(y, before) and torch.equal(x.detach(), before)
    y.sum().backward()
    assert torch.equal(x.grad, torch.full((2, 3), 2.0))      # partial input gradients were summed


def test_reduce_from_region_backward_is_identity_and_buffer_choice_decides_aliasing():
    x = torch.ones(2, 2)
    leaf = torch.ones(2, 2, requires_grad=True)
    out = M._ReduceFromTPRegion.apply(leaf * 1.0, None, _Doubling(), None)
    out.sum().backward()
    assert torch.equal(leaf.grad, torch.ones(2, 2))           # no collective, no scaling in backward
    inplace = M._ReduceFromTPRegion.apply(x, None, _Doubling(), None)
    assert inplace.data_ptr() == x.data_ptr() and torch.equal(x, torch.full((2, 2), 2.0))
    buffers = P.CommunicationBuffer()
    y = torch.ones(2, 2)
    staged = M._ReduceFromTPRegion.apply(y, None, _Doubling(), buffers)
    assert staged.data_ptr() != y.data_ptr() and torch.equal(y, torch.ones(2, 2)) and torch.equal(staged, 2 * y)


def test_backward_of_copy_to_region_uses_the_buffer_when_given():
    buffers = P.CommunicationBuffer()
    x = torch.ones(3, requires_grad=True)
    M._CopyToTPRegion.apply(x, None, _Doubling(), buffers).sum().backward()
    cached = buffers.get_buffer((3,), torch.float32, torch.device("cpu"))
    assert torch.equal(cached, torch.full((3,), 2.0)) and torch.equal(x.grad, cached)


def test_async_collectives_are_waited_for_before_the_result_is_used():
    lazy = _Doubling(lazy=True)
    out = M._ReduceFromTPRegion.apply(torch.ones(4), None, lazy, None)
    assert lazy.pending == [] and torch.equal(out, torch.full((4,), 2.0))
    x = torch.ones(4, requires_grad=True)
    M._CopyToTPRegion.apply(x, None, lazy, None).sum().backward()
    assert lazy.pending == [] and torch.equal(x.grad, torch.full((4,), 2.0))


# ------------------------------------------------------ communication buffer --
def test_communication_buffer_is_keyed_by_shape_dtype_and_device():
    buffers = P.CommunicationBuffer()
    a = buffers.get_buffer((2, 3), torch.float32, torch.device("cpu"))
    assert buffers.get_buffer([2, 3], torch.float32, "cpu") is a
    assert buffers.get_buffer((3, 2), torch.float32, torch.device("cpu")) is not a
    assert buffers.get_buffer((2, 3), torch.bfloat16, torch.device("cpu")) is not a


# ------------------------------------------------------------ shard helpers --
def test_shard_helpers_reject_indivisible_sizes_and_pass_none_bias_through():
    w = torch.randn(6, 4)
    with pytest.raises(ValueError, match="not divisible"):
        P.column_shard(w, None, 0, 4)
    with pytest.raises(ValueError, match="not divisible"):
        P.row_shard(w, None, 0, 3)
    with pytest.raises(ValueError, match="sum"):
        P.blockwise_column_shard(w, None, 0, 2, (4, 4))
    with pytest.raises(ValueError, match="block_sizes"):
        P.blockwise_column_shard(w, None, 0, 2, (3, 3))
    ws, bs = P.column_shard(w, None, 1, 2)
    assert bs is None and torch.equal(ws, w[3:])
    wr, br = P.row_shard(w, torch.ones(6), 1, 2)
    assert torch.equal(wr, w[:, 2:]) and torch.equal(br, torch.ones(6))      # row bias stays whole


def test_fused_qkv_shards_keep_q_k_v_blocks_together_per_rank():
    q_dim, kv_dim, hidden = 8, 4, 5
    w = torch.arange((q_dim + 2 * kv_dim) * hidden, dtype=torch.float32).view(-1, hidden)
    shards = [P.fused_qkv_column_shard(w, None, r, 2, q_dim, kv_dim)[0] for r in range(2)]
    for r, s in enumerate(shards):
        want = torch.cat([w[r * 4:(r + 1) * 4], w[8 + r * 2: 8 + (r + 1) * 2], w[12 + r * 2: 12 + (r + 1) * 2]])
        assert torch.equal(s, want)


# ------------------------------------------------------------------ layers --
def test_parallel_linears_expose_the_reference_attributes_and_local_shapes():
    w, b = torch.randn(8, 6), torch.randn(8)
    col = P.ColumnParallelLinear(w, b, 1, 2, "G", "B")
    row = P.RowParallelLinear(w, b, 1, 2, "G", "B", sequence_parallel=False)
    for layer in (col, row):
        assert (layer.tp_rank, layer.tp_size, layer.group, layer.backend) == (1, 2, "G", "B")
        assert isinstance(layer.buffer_manager, P.CommunicationBuffer) and layer.sequence_parallel is False
    assert col.weight.shape == (4, 6) and col.bias.shape == (4,)
    assert row.weight.shape == (8, 3) and row.bias.shape == (8,)
    local = P.ColumnParallelLinear(w[:4], b[:4], 0, 2, None, None, weight_is_local=True)
    assert torch.equal(local.weight.data, w[:4])


def test_row_parallel_bias_is_added_once_after_the_reduction():
    torch.manual_seed(0)
    x, w, b = torch.randn(3, 8), torch.randn(4, 8), torch.randn(4)

    def rank_fn(rank, be):
        layer = P.RowParallelLinear(w, b, rank, 2, None, be)
        return layer(x[:, rank * 4:(rank + 1) * 4])

    for out in run_ranks(2, rank_fn):
        assert torch.allclose(out, F.linear(x, w, b), atol=1e-5)
    single = P.RowParallelLinear(w, b, 0, 1, None, None)
    assert torch.allclose(single(x), F.linear(x, w, b), atol=1e-6)


# ------------------------------------------------------------ layout rules --
def test_parallel_config_accepts_and_rejects_what_the_reference_does():
    cfg = P.ParallelConfig(tensor_parallel_size=2, pipeline_parallel_size=2)
    assert cfg.product_without_dp() == 4 and cfg.resolved_data_parallel_size(8) == 2
    cfg.validate(8)
    with pytest.raises(ValueError, match="not divisible"):
        cfg.resolved_data_parallel_size(6)
    with pytest.raises(ValueError, match="inconsistent"):
        P.ParallelConfig(tensor_parallel_size=2, data_parallel_size=3).validate(4)
    with pytest.raises(ValueError, match="sequence_parallel is not supported"):
        P.ParallelConfig(tensor_parallel_size=2, context_parallel_size=2, sequence_parallel=True).validate(4)
    with pytest.raises(ValueError, match="pipeline_parallel is not supported"):
        P.ParallelConfig(pipeline_parallel_size=2, context_parallel_size=2).validate(4)
    with pytest.raises(ValueError, match=">= 1"):
        P.ParallelConfig(tensor_parallel_size=0).validate(1)
    with pytest.raises(Exception):
        cfg.tensor_parallel_size = 4                           # frozen


@pytest.mark.parametrize("order", ["tp-cp-dp-pp", "pp-tp-cp-dp", "dp-tp-pp-cp"])
def test_rank_generator_groups_partition_the_world_and_round_trip(order):
    gen = P.RankGenerator(tp=2, dp=2, pp=2, cp=2, order=order)
    assert gen.world_size == 16
    for token in ("tp", "dp", "pp", "cp", "dp-cp", "tp-pp"):
        groups = gen.get_ranks(token)
        flat = sorted(r for g in groups for r in g)
        assert flat == list(range(16))                        # every rank in exactly one group
        width = 1
        for part in token.split("-"):
            width *= 2
        assert all(len(g) == width for g in groups)
    for rank in range(16):
        assert gen.encode(gen.decode(rank)) == rank
    fastest = order.split("-")[0]
    assert gen.get_ranks(fastest)[0] == [0, 1]                # the first dimension of the order is contiguous


def test_reduce_from_tp_region_takes_a_leaf_that_requires_grad():
    """The in-place reduction may be applied to a leaf tensor that requires grad (the
    reference's function allows it); backward is the identity."""
    from nano_megatron_b200.parallel.mappings import _ReduceFromTPRegion

    class _Sum1:
        def all_reduce(self, tensor, *, group=None, op="sum", async_op=False):
            return None

    x = torch.randn(3, 4, requires_grad=True)
    y = _ReduceFromTPRegion.apply(x, None, _Sum1())
    y.sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))
    a = torch.randn(3, 4, requires_grad=True)
    z = _ReduceFromTPRegion.apply(a * 2.0, None, _Sum1())          # the usual case: an activation
    z.sum().backward()
    assert torch.equal(a.grad, torch.full_like(a, 2.0))
