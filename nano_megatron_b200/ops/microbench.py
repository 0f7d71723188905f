"""Per-kernel micro-benchmarks with roofline fractions.

    python -m nano_megatron_b200.ops.microbench gemm --m 4096 --n 4096 --k 1024
    python -m nano_megatron_b200.ops.microbench attn --batch 2 --seq 2048 --heads 16 --dim 64
    python -m nano_megatron_b200.ops.microbench norm | ce | adamw | all

Every kernel is timed with CUDA events after warm-up; between timed launches a
buffer larger than the L2 cache is written so that inputs come from HBM.  The
fractions are against the measured copy bandwidth / cuBLAS throughput of the
machine (``MEASURED_PEAKS.json`` when present).  The same commands are what the
profiler captures are taken from (one kernel, a handful of launches).
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from ..utils.metrics import measured_peaks
from . import kernels, native
from .attention import attn_bwd, attn_fwd
from .gemm import EPI_GELU, gemm_bf16


def _timed(fn, iters: int, flush: bool = True) -> float:
    """Median microseconds per call."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    scratch = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    times = []
    for _ in range(iters):
        if scratch is not None:
            scratch.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    return times[len(times) // 2]


def _report(name: str, us: float, flops: float = 0.0, nbytes: float = 0.0) -> None:
    peaks = measured_peaks()
    parts = [f"{name}: {us:9.1f} us"]
    if flops:
        tf = flops / us / 1e6
        parts.append(f"{tf:7.1f} TFLOP/s ({tf / peaks['bf16_tflops']:.2f} of {peaks['source']} cuBLAS peak)")
    if nbytes:
        gbs = nbytes / us / 1e3
        parts.append(f"{gbs:7.0f} GB/s ({gbs / peaks['hbm_gbs']:.2f} of {peaks['source']} copy bandwidth)")
    print("  ".join(parts), flush=True)


def bench_gemm(args) -> None:
    m, n, k = args.m, args.n, args.k
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    b = torch.randn(n, k, device="cuda").to(torch.bfloat16)
    flops = 2.0 * m * n * k
    _report(f"gemm NT {m}x{n}x{k}", _timed(lambda: gemm_bf16(a, b), args.iters), flops)
    if args.variants:
        bt, at = b.t().contiguous(), a.t().contiguous()
        bias = torch.randn(n, device="cuda").to(torch.bfloat16)
        aux = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        _report("gemm dgrad layout (B MN-major)", _timed(lambda: gemm_bf16(a, bt, b_mn=True), args.iters), flops)
        _report("gemm wgrad layout (A, B MN-major)", _timed(lambda: gemm_bf16(at, bt, a_mn=True, b_mn=True), args.iters), flops)
        _report("gemm + bias + GELU epilogue", _timed(lambda: gemm_bf16(a, b, bias=bias, mode=EPI_GELU, aux_out=aux), args.iters), flops)
        _report("torch.matmul (cuBLAS)", _timed(lambda: torch.matmul(a, b.t()), args.iters), flops)
    if args.epilogues:
        # the epilogue-fused GEMMs of the RoPE / SwiGLU model: QKV + rotary, fc1 + SwiGLU, fc2 dgrad + SwiGLU backward
        from .gemm import EPI_DSWIGLU, EPI_ROPE, EPI_SWIGLU, RopeSpec
        d = 64
        inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, device="cuda").float() / d))
        pos = (torch.arange(m, device="cuda") % 2048).contiguous()
        spec = RopeSpec(RopeSpec.make_table(inv, 2048), pos, (n // 3 * 2) // d * d)
        _report("gemm + rotary epilogue (q, k of a packed QKV)", _timed(lambda: gemm_bf16(a, b, mode=EPI_ROPE, rope=spec), args.iters), flops)
        pre = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        _report("gemm + SwiGLU epilogue (B = [gate; up])", _timed(lambda: gemm_bf16(a, b, mode=EPI_SWIGLU, aux_out=pre), args.iters), flops)
        dy = torch.randn(m, k, device="cuda").to(torch.bfloat16)
        w2 = torch.randn(k, n // 2, device="cuda").to(torch.bfloat16)       # fc2 weight [H, F]
        _report("dgrad gemm + SwiGLU-backward epilogue", _timed(lambda: gemm_bf16(dy, w2, b_mn=True, mode=EPI_DSWIGLU, aux_in=pre), args.iters),
                2.0 * m * (n // 2) * k)


def bench_attn(args) -> None:
    b, s, h, d = args.batch, args.seq, args.heads, args.dim
    qkv = torch.randn(b, s, 3 * h * d, device="cuda").to(torch.bfloat16)
    q = qkv[..., : h * d].view(b, s, h, d)
    k = qkv[..., h * d: 2 * h * d].view(b, s, h, d)
    v = qkv[..., 2 * h * d:].view(b, s, h, d)
    scale = 1.0 / math.sqrt(d)
    out, lse = attn_fwd(q, [k], [v], scale)
    g = torch.randn_like(out)
    fwd_flops = 4.0 * b * h * s * s * d / 2
    _report(f"attention fwd b{b} s{s} h{h} d{d}", _timed(lambda: attn_fwd(q, [k], [v], scale), args.iters), fwd_flops)
    _report("attention bwd (prep + main + dq store)", _timed(lambda: attn_bwd(q, [k], [v], out, g, lse, scale), args.iters),
            2.5 * fwd_flops)
    if args.library:
        _bench_library_attention(args, qkv, g, fwd_flops)


def _bench_library_attention(args, qkv, g, fwd_flops) -> None:
    """The same workload through the flash-attn package, as a yardstick only (it is not
    on any path of this framework)."""
    try:
        from flash_attn import flash_attn_func
    except Exception as exc:  # not installed: say so and carry on
        print(f"flash-attn not importable: {exc}", flush=True)
        return
    b, s, h, d = args.batch, args.seq, args.heads, args.dim
    q, k, v = (t.contiguous().requires_grad_(True) for t in qkv.view(b, s, 3, h, d).unbind(2))
    scale = 1.0 / math.sqrt(d)
    _report("flash-attn (library) fwd", _timed(lambda: flash_attn_func(q, k, v, softmax_scale=scale, causal=True), args.iters),
            fwd_flops)
    out = flash_attn_func(q, k, v, softmax_scale=scale, causal=True)
    _report("flash-attn (library) bwd", _timed(lambda: torch.autograd.grad(out, (q, k, v), g, retain_graph=True), args.iters),
            2.5 * fwd_flops)


def bench_norm(args) -> None:
    r, h = args.rows, args.hidden
    x = torch.randn(r, h, device="cuda").to(torch.bfloat16)
    w = torch.ones(h, device="cuda", dtype=torch.bfloat16)
    bias = torch.zeros(h, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn_like(x)
    _, mean, rstd = kernels.norm_fwd(x, w, bias, 1e-5, False)
    _report(f"layernorm fwd {r}x{h}", _timed(lambda: kernels.norm_fwd(x, w, bias, 1e-5, False), args.iters), nbytes=4.0 * r * h)
    _report("layernorm bwd (dx, dgamma, dbeta)", _timed(lambda: kernels.norm_bwd(dy, x, w, mean, rstd, False), args.iters),
            nbytes=6.0 * r * h)
    _report("bias-gradient column sum", _timed(lambda: kernels.col_sum(dy), args.iters), nbytes=2.0 * r * h)


def bench_ce(args) -> None:
    r, v = args.rows, args.vocab
    logits = torch.randn(r, v, device="cuda").to(torch.bfloat16)
    tgt = torch.randint(0, v, (r,), device="cuda")
    stats = kernels.ce_stats(logits, tgt, 0)
    lse, _, _ = kernels.ce_combine(stats.unsqueeze(0), tgt, -100)
    gs = torch.ones(1, device="cuda")
    dl = torch.empty_like(logits)
    ex = kernels.CeExchange(r, logits.device)
    _report(f"cross-entropy forward, one launch {r}x{v}",
            _timed(lambda: kernels.ce_forward_fused(logits, tgt, 0, -100, ex), args.iters), nbytes=2.0 * r * v)
    _report(f"cross-entropy stats (two-pass kernel of the NCCL path) {r}x{v}",
            _timed(lambda: kernels.ce_stats(logits, tgt, 0), args.iters), nbytes=2.0 * r * v)
    _report("cross-entropy backward", _timed(lambda: kernels.ce_bwd(logits, tgt, 0, -100, lse, gs, out=dl), args.iters),
            nbytes=4.0 * r * v)


def bench_adamw(args) -> None:
    from ..reference.optimizer import AdamW

    n = args.params
    p = torch.nn.Parameter(torch.randn(n, device="cuda").to(torch.bfloat16))
    p.grad = torch.randn(n, device="cuda").to(torch.bfloat16)
    opt = AdamW([("p", p)], lr=1e-4, weight_decay=0.01)
    opt.step()
    _report(f"fused AdamW {n / 1e6:.0f}M bf16 params", _timed(opt.step, args.iters), nbytes=22.0 * n)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("kernel", choices=["gemm", "attn", "norm", "ce", "adamw", "all"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=1024)
    ap.add_argument("--variants", action="store_true")
    ap.add_argument("--epilogues", action="store_true", help="gemm: also time the rotary / SwiGLU epilogue GEMMs")
    ap.add_argument("--library", action="store_true", help="attn: also time the flash-attn package on the same workload")
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--vocab", type=int, default=50304)
    ap.add_argument("--params", type=int, default=64 * 1024 * 1024)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("no CUDA device")
        return 1
    todo = ["gemm", "attn", "norm", "ce", "adamw"] if args.kernel == "all" else [args.kernel]
    for name in todo:
        globals()[f"bench_{name}"](args)
    torch.cuda.synchronize()
    native.check_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())
