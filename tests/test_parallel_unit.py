"""Single-process tests of topology, TP/SP/CP operators, vocab-parallel CE,
attention backends, buckets and DDP (fakes and world-size-1 Gloo groups)."""
from __future__ import annotations

import dataclasses
import os
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.nn.functional as F

import nano_megatron_b200.parallel as P
from nano_megatron_b200.distributed import DistributedDataParallel, GradBucket, TorchDistBackend, build_buckets, \
    reduce_op_from_string
from nano_megatron_b200.distributed.backend import CommBackend
from nano_megatron_b200.parallel import mappings as M
from nano_megatron_b200.parallel.attention_backend import _online_softmax_combine
from nano_megatron_b200.parallel.context_parallel import _GatherFromContextParallelRegion
from nano_megatron_b200.reference import shifted_cross_entropy
from tests._dist_utils import port_for


# ------------------------------------------------------------------ topology --
def test_rank_generator_tables():
    g = P.RankGenerator(tp=2, dp=2, pp=2)
    assert g.get_ranks("tp") == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert g.get_ranks("dp") == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert g.get_ranks("pp") == [[0, 4], [1, 5], [2, 6], [3, 7]]
    g = P.RankGenerator(tp=2, dp=2, pp=1, cp=2)
    assert g.get_ranks("cp") == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert g.get_ranks("dp-cp") == [[0, 2, 4, 6], [1, 3, 5, 7]]
    for r in range(g.world_size):
        assert g.encode(g.decode(r)) == r
    with pytest.raises(ValueError):
        P.RankGenerator(tp=0, dp=1, pp=1)
    with pytest.raises(RuntimeError):
        P.RankGenerator(tp=2, dp=1, pp=1, order="dp-pp")


def test_parallel_config_rules():
    cfg = P.ParallelConfig(tensor_parallel_size=2, pipeline_parallel_size=2)
    assert cfg.product_without_dp() == 4 and cfg.resolved_data_parallel_size(8) == 2
    cfg.validate(8)
    with pytest.raises(ValueError):
        cfg.resolved_data_parallel_size(6)
    with pytest.raises(ValueError):
        P.ParallelConfig(tensor_parallel_size=2, data_parallel_size=3).validate(8)
    with pytest.raises(ValueError, match="sequence_parallel"):
        P.ParallelConfig(tensor_parallel_size=2, context_parallel_size=2, sequence_parallel=True).validate(4)
    with pytest.raises(ValueError, match="pipeline_parallel"):
        P.ParallelConfig(pipeline_parallel_size=2, context_parallel_size=2).validate(4)
    with pytest.raises(ValueError):
        P.ParallelConfig(tensor_parallel_size=0).validate(1)
    with pytest.raises(dataclasses.FrozenInstanceError):
        cfg.tensor_parallel_size = 4


def _fake_ctx(**kw):
    base = dict(tensor_parallel_size=1, tensor_parallel_rank=0, context_parallel_size=1, context_parallel_rank=0,
                data_parallel_size=1, data_parallel_rank=0, pipeline_parallel_size=1, pipeline_parallel_rank=0)
    base.update(kw)
    return SimpleNamespace(**base)


def test_pipeline_neighbour_helpers():
    ctx = _fake_ctx(tensor_parallel_size=2, tensor_parallel_rank=1, data_parallel_size=2, data_parallel_rank=1,
                    pipeline_parallel_size=2, pipeline_parallel_rank=0)
    assert P.is_pipeline_first_stage(ctx) and not P.is_pipeline_last_stage(ctx)
    assert P.pipeline_prev_rank(ctx) is None
    assert P.pipeline_next_rank(ctx) == 1 + 2 * (0 + 1 * (1 + 2 * 1))
    last = _fake_ctx(pipeline_parallel_size=4, pipeline_parallel_rank=3)
    assert P.pipeline_next_rank(last) is None and P.pipeline_prev_rank(last) == 2
    assert P.pipeline_prev_rank(_fake_ctx()) is None and P.pipeline_next_rank(_fake_ctx()) is None


@pytest.fixture
def world1(monkeypatch, request):
    """World-size-1 Gloo process group + parallel context, torn down afterwards."""
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", str(port_for(request.node.nodeid)))
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.delenv("LOCAL_RANK", raising=False)
    ctx = P.initialize_parallel(P.ParallelConfig(), dist_backend="gloo")
    yield ctx
    P.destroy_parallel()


def test_context_world1(world1):
    ctx = world1
    assert ctx.world_size == 1 and ctx.rank == 0 and ctx.tensor_parallel_size == 1
    assert P.is_parallel_initialized() and P.get_parallel_context() is ctx
    assert isinstance(ctx.backend, TorchDistBackend) and isinstance(ctx.backend, CommBackend)
    with pytest.raises(RuntimeError, match="already initialized"):
        P.initialize_parallel(P.ParallelConfig())
    sp = dataclasses.replace(ctx, sequence_parallel=True)
    assert sp.sequence_parallel and sp.tensor_parallel_group is ctx.tensor_parallel_group
    P.destroy_parallel()
    assert not P.is_parallel_initialized()
    with pytest.raises(RuntimeError):
        P.get_parallel_context()
    assert not dist.is_initialized()
    P.initialize_parallel(P.ParallelConfig(), dist_backend="gloo")  # re-init works


def test_reduce_op_strings():
    assert reduce_op_from_string("SUM") == dist.ReduceOp.SUM
    with pytest.raises(ValueError):
        reduce_op_from_string("avg")


# ------------------------------------------------------------ TP / SP at t=1 --
def test_linears_equal_f_linear_at_tp1(world1):
    ctx = world1
    torch.manual_seed(0)
    w, b = torch.randn(12, 8), torch.randn(12)
    x = torch.randn(2, 5, 8, requires_grad=True)
    col = P.ColumnParallelLinear(w, b, 0, 1, ctx.tensor_parallel_group, ctx.backend)
    assert torch.equal(col(x), F.linear(x, w, b))
    w2, b2 = torch.randn(8, 12), torch.randn(8)
    row = P.RowParallelLinear(w2, b2, 0, 1, ctx.tensor_parallel_group, ctx.backend)
    h = torch.randn(2, 5, 12)
    assert torch.equal(row(h), F.linear(h, w2, b2))
    res = torch.randn(2, 5, 8)
    assert torch.allclose(row(h, residual=res), res + F.linear(h, w2, b2))
    y = col(x, gelu=True)
    assert torch.allclose(y, F.gelu(F.linear(x, w, b)), atol=1e-6)
    y.sum().backward()
    assert x.grad is not None and col.weight.grad.shape == w.shape


def test_shard_helpers_reconstruct():
    w, b = torch.arange(48.0).view(12, 4), torch.arange(12.0)
    parts = [P.column_shard(w, b, r, 3) for r in range(3)]
    assert torch.equal(torch.cat([p[0] for p in parts]), w) and torch.equal(torch.cat([p[1] for p in parts]), b)
    rows = [P.row_shard(w, b, r, 2) for r in range(2)]
    assert torch.equal(torch.cat([p[0] for p in rows], dim=1), w) and torch.equal(rows[1][1], b)
    qkv_w = torch.arange(16.0 * 2).view(16, 2)  # Q:8, K:4, V:4
    shards = [P.fused_qkv_column_shard(qkv_w, None, r, 2, 8, 4)[0] for r in range(2)]
    assert torch.equal(shards[1], torch.cat([qkv_w[4:8], qkv_w[10:12], qkv_w[14:16]]))
    with pytest.raises(ValueError):
        P.column_shard(w, b, 0, 5)
    with pytest.raises(ValueError):
        P.blockwise_column_shard(w, None, 0, 2, (6, 5))
    with pytest.raises(ValueError):
        P.blockwise_column_shard(w, None, 0, 4, (6, 6))


class _CountingBackend:
    """Single-rank stand-in that records calls; all-reduce doubles the tensor to
    emulate a two-rank sum of identical values."""

    def __init__(self, double: bool = False):
        self.calls: list[tuple[str, dict]] = []
        self.double = double

    def all_reduce(self, tensor, *, group=None, op="sum", async_op=False):
        self.calls.append(("all_reduce", {"op": op, "async_op": async_op, "numel": tensor.numel()}))
        if self.double and op == "sum":
            tensor.mul_(2)
        return tensor

    def broadcast(self, tensor, src, *, group=None):
        self.calls.append(("broadcast", {"numel": tensor.numel()}))
        return tensor

    def all_gather_into_tensor(self, output, input, *, group=None):
        self.calls.append(("all_gather_into_tensor", {}))
        n = output.shape[0] // input.shape[0] if output.dim() == input.dim() else output.shape[0]
        output.copy_(torch.cat([input] * n) if output.dim() == input.dim() else input.unsqueeze(0).expand_as(output))
        return output

    def reduce_scatter(self, output, input_list, *, group=None, op="sum"):
        self.calls.append(("reduce_scatter", {}))
        output.copy_(sum(input_list))
        return output

    def count(self, name):
        return sum(1 for n, _ in self.calls if n == name)


def test_tp_region_ops_call_async_all_reduce_once():
    be = _CountingBackend()
    x = torch.ones(2, 3)
    out = M._ReduceFromTPRegion.apply(x, None, be, None)
    assert out.data_ptr() == x.data_ptr()  # in place without a buffer
    assert be.calls == [("all_reduce", {"op": "sum", "async_op": True, "numel": 6})]
    buffers = P.CommunicationBuffer()
    out2 = M._ReduceFromTPRegion.apply(x, None, be, buffers)
    assert out2.data_ptr() == buffers.get_buffer(x.shape, x.dtype, x.device).data_ptr() != x.data_ptr()
    be2 = _CountingBackend()
    leaf = torch.ones(2, 3, requires_grad=True)
    M._CopyToTPRegion.apply(leaf, None, be2, None).sum().backward()
    assert be2.count("all_reduce") == 1 and be2.calls[0][1]["async_op"] is True


def test_sequence_parallel_ops_identity_at_tp1_and_shape_checks():
    be = _CountingBackend()
    x = torch.randn(2, 6, 4)
    for fn in (P.scatter_to_sequence_parallel_region, P.gather_from_sequence_parallel_region,
               P.reduce_scatter_to_sequence_parallel_region):
        assert fn(x, None, be, 0, 1).data_ptr() == x.data_ptr()
    assert be.calls == []
    assert torch.equal(P.scatter_to_sequence_parallel_region(x, None, be, 1, 2), x[:, 3:])
    with pytest.raises(ValueError):
        P.scatter_to_sequence_parallel_region(x, None, be, 0, 4)
    with pytest.raises(ValueError):
        P.scatter_to_sequence_parallel_region(torch.randn(5), None, be, 0, 5)


def test_sp_replicated_grads_are_reduced_once_per_backward():
    be = _CountingBackend(double=True)
    a, b = torch.nn.Parameter(torch.ones(3)), torch.nn.Parameter(torch.ones(3))
    for p in (a, b):
        P.register_sequence_parallel_grad_allreduce(p, "g", be)
    (a * 2 + b * 3).sum().backward()
    assert be.count("all_reduce") == 1                      # one coalesced collective for both
    assert torch.equal(a.grad, torch.full((3,), 4.0)) and torch.equal(b.grad, torch.full((3,), 6.0))
    (a * 2 + b * 3).sum().backward()                        # accumulation stays correct
    assert torch.equal(a.grad, torch.full((3,), 8.0))


# ------------------------------------------------------------------ CP ops --
class _Forbidden:
    def __getattr__(self, name):
        raise AssertionError(f"collective {name} must not be called")


def test_cp_ops_single_rank_and_simulated_rank():
    assert P.local_sequence_range(1, 4, 16) == (4, 8)
    with pytest.raises(ValueError):
        P.local_sequence_range(0, 3, 16)
    with pytest.raises(ValueError):
        P.local_sequence_range(4, 4, 16)
    x = torch.randn(2, 8, 3, requires_grad=True)
    assert P.scatter_to_context_parallel_region(x, None, _Forbidden(), 0, 1).data_ptr() == x.data_ptr()
    shard = P.scatter_to_context_parallel_region(x, None, _Forbidden(), 1, 2, seq_dim=1)
    assert torch.equal(shard, x[:, 4:])
    shard.sum().backward()                                   # zero padding, no collective
    assert torch.equal(x.grad[:, :4], torch.zeros(2, 4, 3)) and torch.equal(x.grad[:, 4:], torch.ones(2, 4, 3))
    with pytest.raises(ValueError):
        P.gather_from_context_parallel_region(x, None, _Forbidden(), 0, 2, grad_op="mean")


def test_cp_gather_uses_one_single_buffer_collective():
    be = _CountingBackend()
    x = torch.randn(2, 3, 4, 5, requires_grad=True)          # [B, h, S_loc, d]
    full = P.gather_from_context_parallel_region(x, None, be, 0, 2, seq_dim=2)
    assert full.shape == (2, 3, 8, 5) and be.count("all_gather_into_tensor") == 1
    assert torch.equal(full[:, :, :4], x) and torch.equal(full[:, :, 4:], x)
    full.sum().backward()
    assert be.count("reduce_scatter") == 1 and torch.equal(x.grad, torch.full_like(x, 2.0))
    y = torch.randn(2, 8, 4, requires_grad=True)
    out = _GatherFromContextParallelRegion.apply(y, None, be, 1, 2, 1, "split")
    (out * torch.arange(16.0).view(1, 16, 1)).sum().backward()
    assert torch.equal(y.grad[0, :, 0], torch.arange(8.0, 16.0))


def test_cp_causal_scores_match_full_rows():
    q, k = torch.randn(1, 2, 8, 4), torch.randn(1, 2, 8, 4)
    from nano_megatron_b200.reference.layers import causal_attn_scores
    full = causal_attn_scores(q, k, 0.5)
    part = P.causal_attn_scores_cp(q[:, :, 4:], k, 0.5, query_start=4)
    assert torch.equal(part, full[:, :, 4:])


# ------------------------------------------------------------- vocab CE etc. --
class _IdentityBackend:
    def all_reduce(self, tensor, *, group=None, op="sum", async_op=False):
        return tensor


def test_vocab_parallel_ce_matches_reference_loss_and_grads():
    torch.manual_seed(0)
    logits = torch.randn(2, 6, 10, requires_grad=True)
    labels = torch.randint(0, 10, (2, 6))
    labels[0, 3] = -100
    mine = P.vocab_parallel_cross_entropy(logits, labels, vocab_start_index=0, vocab_end_index=10, group=None,
                                          backend=_IdentityBackend())
    ref_in = logits.detach().clone().requires_grad_(True)
    want = shifted_cross_entropy(ref_in, labels)
    assert torch.allclose(mine, want, atol=1e-6)
    mine.backward()
    want.backward()
    assert torch.allclose(logits.grad, ref_in.grad, atol=1e-6)
    all_ignored = torch.full((2, 6), -100)
    zero = P.vocab_parallel_cross_entropy(logits, all_ignored, vocab_start_index=0, vocab_end_index=10, group=None,
                                          backend=_IdentityBackend())
    assert zero.item() == 0.0 and zero.requires_grad
    assert P.vocab_range_from_global(1, 4, 16) == (4, 8)
    with pytest.raises(ValueError):
        P.vocab_range_from_global(0, 3, 16)


def test_vocab_embedding_masks_foreign_ids():
    w = torch.arange(12.0).view(6, 2)
    emb = P.VocabParallelEmbedding(6, 2, tp_rank=1, tp_size=2, group=None, backend=_IdentityBackend(), weight=w)
    assert (emb.vocab_start_index, emb.vocab_end_index) == (3, 6)
    out = emb(torch.tensor([[0, 3, 5]]))
    assert torch.equal(out[0, 0], torch.zeros(2)) and torch.equal(out[0, 1], w[3]) and torch.equal(out[0, 2], w[5])


def test_attention_backend_resolution_and_unfused_maths():
    cpu = torch.device("cpu")
    assert P.resolve_attention_backend(requested="auto", dtype=torch.float32, device=cpu) == "unfused"
    assert P.resolve_attention_backend(requested="flash", dtype=torch.bfloat16, device=cpu,
                                       return_activations=True) == "unfused"
    with pytest.raises(RuntimeError):
        P.resolve_attention_backend(requested="flash", dtype=torch.float32, device=cpu)
    with pytest.raises(ValueError):
        P.resolve_attention_backend(requested="fast", dtype=torch.float32, device=cpu)
    q, k, v = (torch.randn(1, 2, 6, 4) for _ in range(3))
    want = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=0.5)
    assert torch.allclose(P.unfused_causal_attention(q, k, v, scale=0.5), want, atol=1e-6)
    part = P.unfused_causal_attention(q[:, :, 3:], k, v, scale=0.5, query_start=3)
    assert torch.allclose(part, want[:, :, 3:], atol=1e-6)
    with pytest.raises(ValueError):
        P.unfused_causal_attention(q[:, :, 3:], k, v, scale=0.5)


def test_online_softmax_combine_equals_full_softmax():
    torch.manual_seed(0)
    s = torch.randn(1, 2, 5, 8)                               # [B,h,Sq,Sk]
    v = torch.randn(1, 2, 8, 4)
    full = torch.softmax(s, -1) @ v
    outs, lses = [], []
    for sl in (slice(0, 3), slice(3, 8)):
        outs.append((torch.softmax(s[..., sl], -1) @ v[:, :, sl]).transpose(1, 2))
        lses.append(torch.logsumexp(s[..., sl], -1))
    out, lse = _online_softmax_combine(outs[0], lses[0], outs[1], lses[1])
    assert torch.allclose(out.transpose(1, 2), full, atol=1e-6)
    assert torch.allclose(lse, torch.logsumexp(s, -1), atol=1e-6)


# ---------------------------------------------------------- buckets and DDP --
def _mlp():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.ReLU(), torch.nn.Linear(8, 2))


def test_build_buckets_order_cap_and_dtype_split():
    net = _mlp()
    buckets = build_buckets(net, bucket_cap_mb=25.0)
    assert len(buckets) == 1 and [p.shape for p in buckets[0].params] == [p.shape for p in reversed(list(net.parameters()))]
    small = build_buckets(net, bucket_cap_mb=1e-5)            # ~10 bytes: every parameter alone
    assert len(small) == 4
    net[2].to(torch.float64)
    assert len(build_buckets(net)) == 2
    with pytest.raises(ValueError):
        build_buckets(net, bucket_cap_mb=0)
    with pytest.raises(ValueError):
        GradBucket([])


def test_bucket_sync_mean_and_pure_cp_divisor():
    net = _mlp()
    net(torch.randn(3, 4)).sum().backward()
    want = [p.grad.clone() for p in reversed(list(net.parameters()))]
    bucket = build_buckets(net)[0]
    be = _CountingBackend(double=True)
    params = bucket.params
    assert not bucket.mark_ready(params[0]) and not bucket.mark_ready(params[0]) and bucket.has_pending_ready
    assert [bucket.mark_ready(p) for p in params[1:]] == [False, False, True]
    bucket.sync(be, None, 2)
    assert bucket.coalesced and be.count("all_reduce") == 1
    for p, w in zip(params, want):
        assert torch.allclose(p.grad, w)                     # (g + g) / 2
    bucket.sync(be, None, 2)
    assert be.count("all_reduce") == 1                       # idempotent until reset
    bucket.reset()
    bucket.sync(be, None, 1, group_size=2)                   # pure CP: sum, divide by 1
    for p, w in zip(params, want):
        assert torch.allclose(p.grad, 2 * w)
    bucket.reset()
    bucket.sync(be, None, 1)                                  # group of one: no collective
    assert be.count("all_reduce") == 2
    with pytest.raises(KeyError):
        bucket.mark_ready(torch.nn.Parameter(torch.zeros(1)))
    params[0].grad = None
    bucket.reset()
    with pytest.raises(RuntimeError, match="grad=None"):
        bucket.sync(be, None, 2)


def test_bucket_persistent_buffer_reduces_in_place():
    net = _mlp()
    bucket = build_buckets(net)[0]
    flat = torch.zeros(bucket.numel())
    bucket.bind_persistent(flat)
    net(torch.randn(3, 4)).sum().backward()
    assert all(p.grad.data_ptr() == p.main_grad.data_ptr() for p in bucket.params)
    before = flat.clone()
    bucket.sync(_CountingBackend(double=True), None, 4, group_size=4)
    assert torch.allclose(flat, before * 2 / 4)


def _ddp_ctx(backend, dp=2, cp=1):
    return SimpleNamespace(backend=backend, data_context_parallel_group="dpcp", data_parallel_size=dp,
                           context_parallel_size=cp, data_parallel_rank=0, context_parallel_rank=0, rank=0)


def test_ddp_no_sync_and_finish_with_fake_backend():
    be = _CountingBackend(double=True)
    net = _mlp()
    ddp = DistributedDataParallel(net, _ddp_ctx(be), bucket_cap_mb=1e-5)
    assert be.count("broadcast") == 1                        # one coalesced broadcast per dtype
    n0 = be.count("all_reduce")
    with ddp.no_sync():
        ddp(torch.randn(3, 4)).sum().backward()
    assert be.count("all_reduce") == n0                      # nothing reduced under no_sync
    ddp(torch.randn(3, 4)).sum().backward()
    assert be.count("all_reduce") == n0 + 4                  # every bucket fired during backward
    ddp.finish_grad_sync()
    ddp.finish_grad_sync()
    assert be.count("all_reduce") == n0 + 4
    with ddp.no_sync():
        ddp(torch.randn(3, 4)).sum().backward()
    ddp.finish_grad_sync()                                   # flushes what no_sync deferred
    assert be.count("all_reduce") == n0 + 8


def test_ddp_world1_matches_bare_module_and_reports_unused(world1):
    ctx = world1
    net, bare = _mlp(), _mlp()
    ddp = DistributedDataParallel(net, ctx)
    x = torch.randn(5, 4)
    ddp(x).sum().backward()
    ddp.finish_grad_sync()
    bare(x).sum().backward()
    for a, b in zip(net.parameters(), bare.parameters()):
        assert torch.equal(a.grad, b.grad)
    ddp.finish_grad_sync()                                   # idempotent
    be = _CountingBackend(double=True)
    half = DistributedDataParallel(_mlp(), _ddp_ctx(be))
    half.module[0](torch.randn(2, 4)).sum().backward()       # second layer unused
    half._sync_done = False
    with pytest.raises(RuntimeError, match="missing grads"):
        half.finish_grad_sync()


def test_torch_backend_wraps_every_protocol_method(world1):
    be = world1.backend
    t = torch.ones(4)
    assert torch.equal(be.all_reduce(t.clone()), t)
    work = be.all_reduce(t.clone(), async_op=True)
    work.wait()
    out = torch.empty(4)
    be.all_gather_into_tensor(out, t)
    assert torch.equal(out, t)
    lst = [torch.empty(4)]
    be.all_gather(lst, t)
    assert torch.equal(lst[0], t)
    rs = torch.empty(4)
    be.reduce_scatter(rs, [t.clone()])
    assert torch.equal(rs, t)
    assert torch.equal(be.broadcast(t.clone(), 0), t)
    be.barrier()


def test_reference_import_paths_and_rank_helpers_exist():
    """``nano_megatron.model`` / ``.model.tp_gpt`` / ``.model.pipeline`` of the reference map to
    the same modules here, and the stride helper of the rank generator is public as there."""
    import nano_megatron_b200.model as alias
    import nano_megatron_b200.model.pipeline as alias_pp
    import nano_megatron_b200.model.tp_gpt as alias_tp
    import nano_megatron_b200.models as models
    from nano_megatron_b200.parallel.rank_generator import prefix_product

    assert alias_tp is models.tp_gpt and alias_pp is models.pipeline
    assert set(alias.__all__) == set(models.__all__) and alias.TPGPT is models.TPGPT
    assert prefix_product([2, 3, 4]) == [1, 2, 6, 24]
    assert prefix_product([], init=5) == [5]
