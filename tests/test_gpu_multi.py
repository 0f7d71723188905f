"""Multi-GPU tests (NCCL + peer-memory kernels), one process per GPU.

Launchers are skipped when fewer GPUs are visible than the case needs.  The
oracle is the fp32 CPU ``ReferenceGPT`` on the global batch.
"""
from __future__ import annotations

import os

import pytest
import torch
import torch.distributed as dist

from tests._dist_utils import launch, run_worker_if_requested

pytestmark = pytest.mark.gpu
HERE = os.path.abspath(__file__)


def _setup(symm=True, **cfg_kw):
    import nano_megatron_b200.parallel as P
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    ctx = P.initialize_parallel(P.ParallelConfig(**cfg_kw), dist_backend="nccl")
    made = {}
    if symm:
        from nano_megatron_b200.distributed.symm_mem import enable_symmetric_memory
        made = enable_symmetric_memory(ctx)
    torch.manual_seed(1234)
    return P, ctx, made


def _finish(P):
    from nano_megatron_b200.ops import native
    torch.cuda.synchronize()
    native.check_status()
    dist.barrier()
    P.destroy_parallel()


def worker_symm_allreduce():
    from nano_megatron_b200.distributed.symm_mem import SymmetricWorkspace
    P, ctx, _ = _setup(symm=False)
    ws = SymmetricWorkspace(dist.group.WORLD)
    n = ws.size
    for dtype, numel in ((torch.bfloat16, 8 * 1000 + 8), (torch.float32, 4 * 77), (torch.bfloat16, 25 * 1024 * 1024 // 2)):
        t = ws.alloc_tensor(numel, dtype)
        for trial in range(3):
            src = (torch.randn(numel, device="cuda") * (ctx.rank + 1 + trial)).to(dtype)
            t.copy_(src)
            ref = src.float().clone()
            dist.all_reduce(ref)
            ws.all_reduce_scale_(t, 1.0 / n)
            torch.cuda.synchronize()
            tol = 3e-2 * ref.abs().max().item() / n if dtype == torch.bfloat16 else 1e-5 * ref.abs().max().item()
            assert (t.float() - ref / n).abs().max().item() <= tol, (dtype, numel, trial)
    ws.barrier()
    # timing vs NCCL for a 25 MiB bf16 bucket
    big = ws.alloc_tensor(25 * 1024 * 1024 // 2, torch.bfloat16)
    plain = torch.zeros_like(big)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            fn()
        b.record(); torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / 20], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    mine = timed(lambda: ws.all_reduce_scale_(big, 0.5))
    nccl = timed(lambda: (dist.all_reduce(plain), plain.div_(2)))
    if ctx.rank == 0:
        print(f"PERF allreduce+scale 25MiB x{n}: peer-kernel {mine*1e3:.1f} us, NCCL+div {nccl*1e3:.1f} us", flush=True)
    _finish(P)


def worker_ddp_symmetric():
    from nano_megatron_b200.distributed import DistributedDataParallel
    P, ctx, made = _setup()
    assert "dp-cp" in made
    torch.manual_seed(5)
    net = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.Tanh(), torch.nn.Linear(256, 32))
    full = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.Tanh(), torch.nn.Linear(256, 32))
    full.load_state_dict(net.state_dict())
    net = net.cuda().to(torch.bfloat16)
    ddp = DistributedDataParallel(net, ctx, bucket_cap_mb=0.02)
    assert all(b.fused_reduce is not None for b in ddp._buckets)
    x = torch.randn(8 * ctx.world_size, 64)
    for step in range(2):
        ddp.zero_grad(); full.zero_grad()
        mine = x[ctx.rank * 8:(ctx.rank + 1) * 8].cuda().to(torch.bfloat16)
        ddp(mine).float().pow(2).mean().backward()
        ddp.finish_grad_sync()
        full(x).pow(2).mean().backward()
        for p, q in zip(net.parameters(), full.parameters()):
            err = (p.grad.float().cpu() - q.grad).abs().max().item()
            assert err < 5e-2 * max(q.grad.abs().max().item(), 1e-3), (step, err)
    _finish(P)


def _gpu_model_worker(knobs, seq=256, batch=2, tol=8e-2, **layout):
    from nano_megatron_b200.distributed import DistributedDataParallel
    from nano_megatron_b200.models import build_tp_gpt_from_reference
    from nano_megatron_b200.reference import ReferenceGPT, ReferenceGPTConfig, seed_all, shifted_cross_entropy
    P, ctx, _ = _setup(**layout)
    seed_all(0)
    cfg = ReferenceGPTConfig(num_layers=2, hidden_size=256, num_heads=4, vocab_size=512, max_seq_len=seq,
                             attn_backend="flash", **knobs)
    ref = ReferenceGPT(cfg)
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() > 1:
                p.mul_(0.5)
    dp = ctx.data_parallel_size
    ids = torch.randint(0, cfg.vocab_size, (batch * dp, seq))
    model = build_tp_gpt_from_reference(ref, ctx).to("cuda", dtype=torch.bfloat16)
    ddp = DistributedDataParallel(model, ctx)
    sl = slice(ctx.data_parallel_rank * batch, (ctx.data_parallel_rank + 1) * batch)
    logits = ddp(ids[sl].cuda())
    loss = model.shifted_cross_entropy(logits, ids[sl].cuda())
    loss.backward()
    ddp.finish_grad_sync()
    torch.cuda.synchronize()
    cpu_cfg = ReferenceGPTConfig(**{**cfg.__dict__, "attn_backend": "unfused"})
    ref.config = cpu_cfg
    for blk in ref.blocks:
        blk.attn.config = cpu_cfg
    ref_loss = shifted_cross_entropy(ref(ids), ids)
    ref_loss.backward()
    mean = loss.detach().float().clone()
    dist.all_reduce(mean, group=ctx.data_context_parallel_group)
    mean /= (dp * ctx.context_parallel_size)
    assert abs(mean.item() - ref_loss.item()) < 3e-2 * abs(ref_loss.item()), (mean.item(), ref_loss.item())
    from tests.test_distributed_gloo import _expected_shard
    ref_grads = {n: p.grad for n, p in ref.named_parameters()}
    for n, p in model.named_parameters():
        want = _expected_shard(n, ref_grads[n], ctx, cfg)
        got = p.grad.float().cpu()
        rel = (got - want).norm().item() / (want.norm().item() + 1e-6)
        assert rel < tol, (n, rel)
    _finish(P)


GPT2 = dict(position_embedding_type="learned_absolute", gated_linear_unit=False, use_bias=True, use_fused_qkv=True)


def worker_tp2_bf16():
    _gpu_model_worker(GPT2, tensor_parallel_size=2)


def worker_sp2_bf16():
    from nano_megatron_b200.ops import fused_tp
    _gpu_model_worker(GPT2, tensor_parallel_size=2, sequence_parallel=True)
    # 2 layers: (qkv, fc1) x 2 + lm_head gathers forward, (out, fc2) x 2 gathers backward, and the mirror image
    assert fused_tp.STATS["allgather_gemm"] >= 9 and fused_tp.STATS["gemm_reduce_scatter"] >= 9, fused_tp.STATS


def worker_dp2_bf16():
    _gpu_model_worker(dict(GPT2, tie_word_embeddings=True))


def worker_cp2_bf16():
    _gpu_model_worker(dict(use_fused_qkv=True, use_bias=True), context_parallel_size=2)


def worker_pp2_bf16():
    from nano_megatron_b200.models import build_pipeline_stage_from_reference
    from nano_megatron_b200.reference import ReferenceGPT, ReferenceGPTConfig, seed_all, shifted_cross_entropy
    from nano_megatron_b200.schedules import forward_backward_1f1b
    P, ctx, _ = _setup(symm=False, pipeline_parallel_size=2)
    seed_all(0)
    cfg = ReferenceGPTConfig(num_layers=4, hidden_size=256, num_heads=4, vocab_size=512, max_seq_len=256,
                             attn_backend="flash", **GPT2)
    ref = ReferenceGPT(cfg)
    ids = torch.randint(0, cfg.vocab_size, (4, 256))
    stage = build_pipeline_stage_from_reference(ref, ctx).to("cuda", dtype=torch.bfloat16)
    loss = forward_backward_1f1b(stage=stage, ctx=ctx, input_ids=ids.cuda(), labels=ids.cuda(), num_microbatches=2)
    torch.cuda.synchronize()
    cpu_cfg = ReferenceGPTConfig(**{**cfg.__dict__, "attn_backend": "unfused"})
    ref.config = cpu_cfg
    for blk in ref.blocks:
        blk.attn.config = cpu_cfg
    ref_loss = shifted_cross_entropy(ref(ids), ids)
    if P.is_pipeline_last_stage(ctx):
        assert abs(loss.item() - ref_loss.item()) < 3e-2 * abs(ref_loss.item())
    _finish(P)


def worker_peer_leaves_between_steps():
    """A rank stops between steps (nothing in flight); the survivor's next
    collective ends with an error from the process-group timeout, not a hang."""
    import datetime
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=10))
    t = torch.ones(4, device="cuda")
    dist.all_reduce(t)
    torch.cuda.synchronize()
    if dist.get_rank() == 1:
        os._exit(0)                      # leaves between steps
    try:
        dist.all_reduce(t)
        torch.cuda.synchronize()
        survived = False
    except Exception:
        survived = True
    print("SURVIVOR_SAW_ERROR" if survived else "SURVIVOR_SAW_NOTHING", flush=True)
    os._exit(0)


CASES = [("worker_symm_allreduce", 2), ("worker_ddp_symmetric", 2), ("worker_tp2_bf16", 2), ("worker_sp2_bf16", 2),
         ("worker_dp2_bf16", 2), ("worker_cp2_bf16", 2), ("worker_pp2_bf16", 2)]


@pytest.mark.parametrize("worker,world", CASES, ids=[f"{w}-{n}" for w, n in CASES])
def test_multi_gpu(worker, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    launch(HERE, worker, world, timeout=300, extra_env={"NCCL_NVLS_ENABLE": "0"})


if __name__ == "__main__":
    run_worker_if_requested(globals())
