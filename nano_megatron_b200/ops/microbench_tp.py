"""Micro-benchmark of the fused tensor/sequence-parallel GEMMs against the
unfused sequence (NCCL collective + GEMM), with roofline fractions.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m nano_megatron_b200.ops.microbench_tp [--batch 2 --seq 2048 --hidden 1024 --ffn 4096]

Every rank runs every operation in lockstep; times are CUDA-event medians with
the L2 flushed between launches, maximum over ranks.  The roofline of a fused
op is the slower of its FLOPs at the measured cuBLAS peak and the bytes it must
move over NVLink at 770 GB/s per direction (measured peer-copy bandwidth); the
fraction printed is that time divided by the measured time.  The reference has
no counterpart (its layers call ``all_gather`` / ``reduce_scatter`` and
``F.linear`` one after the other, nano_megatron/parallel/mappings.py:226-286,
:419, :450).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _timed(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    scratch = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    times = []
    for _ in range(iters):
        scratch.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    t = torch.tensor([times[len(times) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--ffn", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2 or not torch.cuda.is_available():
        print("needs >= 2 ranks with one GPU each (run under torch.distributed.run)")
        return 1
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")

    import nano_megatron_b200.parallel as P
    from ..distributed.symm_mem import enable_symmetric_memory
    from ..utils.metrics import measured_peaks
    from . import native
    from .fused_tp import _place_shard, tp_fused_for
    from .gemm import gemm_bf16

    ctx = P.initialize_parallel(P.ParallelConfig(tensor_parallel_size=world, sequence_parallel=True),
                                dist_backend="nccl")
    enable_symmetric_memory(ctx)
    st = tp_fused_for(ctx.tensor_parallel_group)
    group = ctx.tensor_parallel_group
    peaks = measured_peaks()
    b, s, h, f, t = args.batch, args.seq, args.hidden, args.ffn, world
    rows = b * s

    def report(name: str, us_fused: float, us_plain: float, flops: float, link_bytes: float) -> None:
        if rank != 0:
            return
        t_compute = flops / (peaks["bf16_tflops"] * 1e12) * 1e6
        t_link = link_bytes / (NVLINK_GBS * 1e9) * 1e6
        target = max(t_compute, t_link)
        print(f"{name}: fused {us_fused:7.1f} us | NCCL + GEMM {us_plain:7.1f} us | roofline {target:5.1f} us "
              f"(compute {t_compute:.1f}, link {t_link:.1f}; {peaks['source']} peaks) -> {target / us_fused:.2f} of roofline",
              flush=True)

    # ---- all-gather -> GEMM (column-parallel linear under SP) ----
    for label, n_out in (("qkv", 3 * h // t), ("fc1", f // t)):
        w = (torch.randn(n_out, h, device="cuda") * 0.02).to(torch.bfloat16)
        shard = torch.randn(b, s // t, h, device="cuda").to(torch.bfloat16)
        full = st.gather_buffer(rows, h)
        _place_shard(full, shard, ctx.tensor_parallel_rank, s, t)
        gathered = torch.empty(rows, h, dtype=torch.bfloat16, device="cuda")
        flat = shard.reshape(-1, h).contiguous()

        def fused():
            st.allgather_gemm(full, w, s)

        def plain():
            dist.all_gather_into_tensor(gathered, flat, group=group)
            gemm_bf16(gathered, w)

        report(f"all-gather -> GEMM {label} [{rows} x {n_out} x {h}]", _timed(fused, args.iters),
               _timed(plain, args.iters), 2.0 * rows * n_out * h, rows * h * 2.0 * (t - 1) / t)

    # ---- GEMM -> reduce-scatter (row-parallel linear under SP) ----
    for label, k_in in (("proj", h // t), ("fc2", f // t)):
        w = (torch.randn(h, k_in, device="cuda") * 0.02).to(torch.bfloat16)
        a = torch.randn(rows, k_in, device="cuda").to(torch.bfloat16)
        out = torch.empty(rows // t, h, dtype=torch.bfloat16, device="cuda")

        def fused():
            st.gemm_reduce_scatter(a, w, s)

        def plain():
            partial = gemm_bf16(a, w)
            dist.reduce_scatter_tensor(out, partial, group=group)

        report(f"GEMM -> reduce-scatter {label} [{rows} x {h} x {k_in}]", _timed(fused, args.iters),
               _timed(plain, args.iters), 2.0 * rows * h * k_in, rows * h * 2.0 * (t - 1) / t)

    torch.cuda.synchronize()
    native.check_status()
    dist.barrier()
    P.destroy_parallel()
    return 0


if __name__ == "__main__":
    sys.exit(main())
