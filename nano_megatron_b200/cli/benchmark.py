"""Benchmark driver and report writer.

The reference ships one script per parallelism mode
(``scripts/benchmark_{tp,dp,cp,pp}.py``): each times its own framework and
Megatron-LM, collects a ``BenchmarkResult`` (tokens/s, peak memory, step time)
per framework and can write a markdown report
(``scripts/benchmark_tp.py:402-487``).  Here one command covers the modes:

    python -m nano_megatron_b200.cli.benchmark --gpus 2 --modes dp tp cp --impls b200 reference \
        --report performance.md

It runs ``bench.py`` (the repository's benchmark program: device-timed,
maximum over ranks) once per mode and implementation under
``torch.distributed.run``, reads the JSON line each run prints, and writes the
same kind of table: framework, mode, model, batch, sequence, tokens/s, peak MB,
step ms -- for the full step (with AdamW) and for the reference's own benchmark
step (forward, backward, gradient sync, zero-grad).  ``--from-json`` builds the
report from saved JSON lines instead of running anything.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
from dataclasses import dataclass
from typing import Iterable, Optional


@dataclass
class BenchmarkResult:
    framework: str
    model_name: str
    parallelism: str
    n_gpus: int
    batch_size: int
    seq_len: int
    tokens_per_sec: float
    memory_mb: float
    avg_step_time_ms: float
    tokens_per_sec_no_optimizer: Optional[float] = None
    step_time_ms_no_optimizer: Optional[float] = None
    tokens_per_sec_e2e: Optional[float] = None


def results_from_json(payload: dict) -> list[BenchmarkResult]:
    """One result for the headline of a ``bench.py`` line plus one per entry under ``modes``."""
    if "unavailable" in payload or "value" not in payload:
        return []
    impl = payload.get("impl", "b200")
    out = []

    def one(cfg: dict, body: dict) -> BenchmarkResult:
        nopt = body.get("step_without_optimizer") or {}
        return BenchmarkResult(
            framework="nano_megatron_b200" if impl == "b200" else impl, model_name=cfg.get("model", "GPT"),
            parallelism=cfg.get("parallelism", "?"), n_gpus=int(payload.get("n_gpus", 1)),
            batch_size=int(cfg.get("global_batch", 0)), seq_len=int(cfg.get("seq_len", 0)),
            tokens_per_sec=float(body["value"]), memory_mb=float(body.get("peak_mem_mb") or 0.0),
            avg_step_time_ms=float(body["ms_per_step"]), tokens_per_sec_no_optimizer=nopt.get("value"),
            step_time_ms_no_optimizer=nopt.get("ms_per_step"), tokens_per_sec_e2e=(body.get("e2e") or {}).get("value"))

    out.append(one(payload["config"], payload))
    for entry in (payload.get("modes") or {}).values():
        if "value" in entry:
            out.append(one(entry["config"], entry))
    return out


def format_result_markdown(r: BenchmarkResult) -> str:
    nopt = f"{r.tokens_per_sec_no_optimizer:,.0f}" if r.tokens_per_sec_no_optimizer else "-"
    nopt_ms = f"{r.step_time_ms_no_optimizer:.2f}" if r.step_time_ms_no_optimizer else "-"
    return (f"| {r.framework} | {r.model_name} | {r.parallelism} | {r.n_gpus} | {r.batch_size} | {r.seq_len} | "
            f"{r.tokens_per_sec:,.0f} | {r.avg_step_time_ms:.2f} | {nopt} | {nopt_ms} | {r.memory_mb:,.0f} |")


def write_performance_md(results: Iterable[BenchmarkResult], output_path: str, *, title: str = "Benchmark report",
                         environment: Optional[dict] = None) -> None:
    results = list(results)
    env = environment or {}
    lines = [f"# {title}", "", "## Test environment", ""]
    lines += [f"- **{k}**: {v}" for k, v in env.items()]
    lines += [f"- **Date**: {datetime.datetime.now().strftime('%Y-%m-%d %H:%M:%S')}", "",
              "## Results", "",
              "tokens/s is the whole job (all GPUs); times are CUDA-event times, maximum over ranks.  "
              "\"no optimizer\" is forward + backward + gradient synchronisation + zero-grad.", "",
              "| Framework | Model | Parallelism | GPUs | Global batch | Seq len | Tokens/s (step with AdamW) | Step ms | "
              "Tokens/s (no optimizer) | Step ms (no optimizer) | Peak memory (MB) |",
              "|---|---|---|---|---|---|---|---|---|---|---|"]
    lines += [format_result_markdown(r) for r in results]
    by_key: dict[tuple, dict[str, BenchmarkResult]] = {}
    for r in results:
        by_key.setdefault((r.model_name, r.parallelism, r.n_gpus, r.batch_size, r.seq_len), {})[r.framework] = r
    ratios = []
    for key, group in by_key.items():
        mine, ref = group.get("nano_megatron_b200"), group.get("reference")
        if mine and ref and ref.tokens_per_sec > 0:
            line = f"- {key[1]} on {key[2]} GPU(s), {key[0]}: {mine.tokens_per_sec / ref.tokens_per_sec:.2f}x with AdamW"
            if mine.tokens_per_sec_no_optimizer and ref.tokens_per_sec_no_optimizer:
                line += f", {mine.tokens_per_sec_no_optimizer / ref.tokens_per_sec_no_optimizer:.2f}x without"
            if ref.memory_mb > 0 and mine.memory_mb > 0:
                line += f"; peak memory {mine.memory_mb / ref.memory_mb:.2f}x"
            ratios.append(line)
    if ratios:
        lines += ["", "## nano_megatron_b200 / reference", ""] + ratios
    with open(output_path, "w") as f:
        f.write("\n".join(lines) + "\n")


def _find_bench(path: Optional[str]) -> str:
    if path:
        return path
    here = os.path.dirname(os.path.abspath(__file__))
    guess = os.path.join(os.path.dirname(os.path.dirname(here)), "bench.py")
    if not os.path.exists(guess):
        raise SystemExit("bench.py not found next to the package; pass --bench-script")
    return guess


def run_bench(bench: str, gpus: int, mode: str, impl: str, steps: int, warmup: int, extra: list[str],
              port: int) -> Optional[dict]:
    cmd = [sys.executable]
    if gpus > 1:
        cmd += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
                "--master-port", str(port)]
    cmd += [bench, "--gpus", str(gpus), "--steps", str(steps), "--warmup", str(warmup), "--mode", mode, "--impl", impl,
            *extra]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    for line in proc.stdout.splitlines():
        if line.startswith("{"):
            return json.loads(line)
    sys.stderr.write(proc.stderr[-2000:])
    return None


def main(argv: Optional[list[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--modes", nargs="+", default=["dp"], choices=["dp", "tp", "cp", "pp"])
    ap.add_argument("--impls", nargs="+", default=["b200"], choices=["b200", "nccl-baseline", "reference"])
    ap.add_argument("--model", default="345m")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--report", default=None, help="markdown file to write")
    ap.add_argument("--from-json", nargs="*", default=None, help="files of saved bench.py JSON lines")
    ap.add_argument("--bench-script", default=None)
    args, extra = ap.parse_known_args(argv)
    results: list[BenchmarkResult] = []
    if args.from_json is not None:
        for path in args.from_json:
            with open(path) as f:
                for line in f:
                    if line.startswith("{"):
                        results += results_from_json(json.loads(line))
    else:
        bench = _find_bench(args.bench_script)
        port = 29700
        for mode in args.modes:
            for impl in args.impls:
                port += 1
                payload = run_bench(bench, args.gpus, mode, impl, args.steps, args.warmup,
                                    ["--model", args.model, *extra], port)
                if payload is None:
                    print(f"{impl} {mode}: no result")
                    continue
                results += results_from_json(payload)
    for r in results:
        print(format_result_markdown(r))
    if args.report:
        import torch
        env = {"PyTorch": torch.__version__, "CUDA": torch.version.cuda}
        if torch.cuda.is_available():
            env["GPU"] = f"{torch.cuda.get_device_name(0)} x {args.gpus}"
        write_performance_md(results, args.report, environment=env)
        print(f"wrote {args.report}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
