"""Micro-benchmark of the fused tensor/sequence-parallel GEMMs against the
unfused sequence (NCCL collective + GEMM), with roofline fractions.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m nano_megatron_b200.ops.microbench_tp [--batch 2 --seq 2048 --hidden 1024 --ffn 4096]

Every rank runs every operation in lockstep.  An operation is timed as a train
of back-to-back launches between one pair of CUDA events (maximum over ranks,
divided by the train length), the launches cycling through enough distinct
input sets that the train's working set exceeds the 126 MB L2.  The fused
kernels are timed twice: launched eagerly like the NCCL + GEMM pair, and as a
captured CUDA graph of the same train (how they run inside a training step,
where the host is out of the picture).  The roofline of a fused op is the
slower of its FLOPs at the measured cuBLAS peak and the bytes it must move over
NVLink at 770 GB/s per direction (measured peer-copy bandwidth); the fraction
printed is that time divided by the measured (graph) time.  The reference has
no counterpart (its layers call ``all_gather`` / ``reduce_scatter`` /
``all_reduce`` and ``F.linear`` one after the other,
nano_megatron/parallel/mappings.py:226-286, :419, :450).
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _train(fn, sets: int, length: int) -> float:
    """us per call of ``fn(i)`` (i = input-set index) in a back-to-back train."""
    for i in range(min(sets, 3)):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    best = None
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        a.record()
        for i in range(length):
            fn(i % sets)
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) * 1e3 / length], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        best = t.item() if best is None else min(best, t.item())
    return float(best)


def _graphed(fn, sets: int, length: int) -> float:
    """The same train captured once into a CUDA graph and replayed."""
    for i in range(min(sets, 3)):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        for i in range(length):
            fn(i % sets)
    torch.cuda.synchronize()
    us = _train(lambda _i: graph.replay(), 1, 4) / length
    del graph
    return us


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--ffn", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=24, help="launches per timed train")
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

    def report(name: str, us_graph: float, us_fused: float, us_plain: float, flops: float, link_bytes: float,
               us_gemm: float = 0.0) -> None:
        if rank != 0:
            return
        if us_gemm:
            name = f"{name} (GEMM alone {us_gemm:.1f} us)"
        t_compute = flops / (peaks["bf16_tflops"] * 1e12) * 1e6
        t_link = link_bytes / (NVLINK_GBS * 1e9) * 1e6
        target = max(t_compute, t_link)
        print(f"{name}: fused {us_graph:6.1f} us in a graph, {us_fused:6.1f} us eager | NCCL + GEMM {us_plain:6.1f} us "
              f"| roofline {target:5.1f} us (compute {t_compute:.1f}, link {t_link:.1f}; {peaks['source']} peaks) "
              f"-> {target / us_graph:.2f} of roofline", flush=True)

    length = args.iters
    # ---- all-gather -> GEMM (column-parallel linear under SP) ----
    for label, n_out in (("qkv", 3 * h // t), ("fc1", f // t)):
        sets = max(2, (160 << 20) // (rows * h * 2) + 1)
        w = (torch.randn(n_out, h, device="cuda") * 0.02).to(torch.bfloat16)
        shard = torch.randn(b, s // t, h, device="cuda").to(torch.bfloat16)
        fulls = [st.gather_buffer(rows, h, owner=("mb", label, i)) for i in range(sets)]
        for full in fulls:
            _place_shard(full, shard, ctx.tensor_parallel_rank, s, t)
        gathered = [torch.empty(rows, h, dtype=torch.bfloat16, device="cuda") for _ in range(sets)]
        flat = shard.reshape(-1, h).contiguous()

        def fused(i):
            st.allgather_gemm(fulls[i], w, s)

        def plain(i):
            dist.all_gather_into_tensor(gathered[i], flat, group=group)
            gemm_bf16(gathered[i], w)

        report(f"all-gather -> GEMM {label} [{rows} x {n_out} x {h}]", _graphed(fused, sets, length),
               _train(fused, sets, length), _train(plain, sets, length), 2.0 * rows * n_out * h,
               rows * h * 2.0 * (t - 1) / t, _graphed(lambda i: gemm_bf16(gathered[i], w), sets, length))

    # ---- GEMM -> reduce-scatter (row-parallel linear under SP), GEMM -> all-reduce (without SP) ----
    for label, k_in in (("proj", h // t), ("fc2", f // t)):
        sets = max(2, (160 << 20) // (rows * k_in * 2) + 1)
        w = (torch.randn(h, k_in, device="cuda") * 0.02).to(torch.bfloat16)
        a = [torch.randn(rows, k_in, device="cuda").to(torch.bfloat16) for _ in range(sets)]
        out = torch.empty(rows // t, h, dtype=torch.bfloat16, device="cuda")
        full_out = torch.empty(rows, h, dtype=torch.bfloat16, device="cuda")

        def fused_rs(i):
            st.gemm_reduce_scatter(a[i], w, s)

        def plain_rs(i):
            partial = gemm_bf16(a[i], w)
            dist.reduce_scatter_tensor(out, partial, group=group)

        def fused_ar(i):
            st.gemm_all_reduce(a[i], w)

        def plain_ar(i):
            gemm_bf16(a[i], w, out=full_out)
            dist.all_reduce(full_out, group=group)

        report(f"GEMM -> reduce-scatter {label} [{rows} x {h} x {k_in}]", _graphed(fused_rs, sets, length),
               _train(fused_rs, sets, length), _train(plain_rs, sets, length), 2.0 * rows * h * k_in,
               rows * h * 2.0 * (t - 1) / t, _graphed(lambda i: gemm_bf16(a[i], w), sets, length))
        if st.all_reduce_supported(rows, h):
            report(f"GEMM -> all-reduce {label} [{rows} x {h} x {k_in}]", _graphed(fused_ar, sets, length),
                   _train(fused_ar, sets, length), _train(plain_ar, sets, length), 2.0 * rows * h * k_in,
                   2.0 * rows * h * 2.0 * (t - 1) / t)

    torch.cuda.synchronize()
    native.check_status()
    dist.barrier()
    P.destroy_parallel()
    return 0


if __name__ == "__main__":
    sys.exit(main())
