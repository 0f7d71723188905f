#!/usr/bin/env python
"""Headline benchmark: GPT training tokens/sec on N GPUs of one node.

    python bench.py --gpus 1 --steps 100 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W [--mode dp|tp|cp|pp] [--impl reference]

The headline step is zero-grad, forward, shifted cross entropy, backward,
gradient synchronisation and an AdamW update, bf16 parameters, synthetic
uniform token ids, random-init weights.  The same JSON line also carries

* ``step_without_optimizer``: the reference's own benchmark step (forward,
  backward, gradient sync, zero-grad; nano_megatron scripts/benchmark_tp.py:182-186,
  benchmark_dp.py:212-223), timed the same way;
* ``peak_mem_mb``: peak device memory of the run (torch allocator peak plus
  symmetric memory), the third column of the reference's benchmark tables;
* ``modes`` (only when no ``--mode`` is given): the other configurations of the
  benchmark suite at the same GPU count -- GPT-760M data parallel, GPT-345M
  tensor + sequence parallel, GPT-1.3B context parallel, the TP x PP (x DP)
  composite with the 1F1B schedule, and the reference's published knob set
  (RoPE, SwiGLU, no bias, untied, vocabulary 51200) -- each with both step
  figures.

Rank 0 prints ONE JSON line.  ``--impl reference`` runs the unmodified
reference package (installed offline into ``baseline/_ref``) through its own
modules for the same steps and configurations.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

T_START = time.time()

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Published by the reference on 4x RTX A6000 (its performance.md), global tok/s,
# bf16 + flash attention, per-rank batch 2 x 2048 (1.3B: 1 x 2048).
PUBLISHED = {
    ("345m", "dp", 2): 33494.0, ("760m", "dp", 2): 19167.0, ("1.3b", "dp", 2): 10211.0,
    ("345m", "tp", 2): 26725.0, ("345m", "tp", 4): 31655.0, ("760m", "tp", 2): 16516.0,
    ("760m", "tp", 4): 20956.0, ("1.3b", "tp", 2): 10852.0, ("1.3b", "tp", 4): 14457.0,
    ("345m", "cp", 2): 20718.0, ("760m", "cp", 2): 12422.0, ("1.3b", "cp", 2): 6420.0,
}

METRIC = "training tokens/sec/box (device-timed, max over ranks), fwd+bwd+grad-sync+AdamW, bf16"


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "nccl-baseline", "reference"],
                    help="b200: this framework; nccl-baseline: this framework's modules on plain NCCL collectives "
                         "(same as --no-symm); reference: the unmodified reference package")
    ap.add_argument("--mode", default=None, choices=["dp", "tp", "cp", "pp", "composite"],
                    help="one configuration only (composite = pp: TP2 x PP2 (x DP2 at 8 GPUs) with the 1F1B "
                         "schedule); without it the headline is dp and the other modes are added under 'modes'")
    ap.add_argument("--model", default="345m", choices=["345m", "760m", "1.3b", "small"])
    ap.add_argument("--knobs", default="gpt2", choices=["gpt2", "published"],
                    help="gpt2: GELU, learned positions, bias, tied, vocabulary 50304; published: the reference's "
                         "benchmark knobs (RoPE, SwiGLU, no bias, untied, vocabulary 51200)")
    ap.add_argument("--batch", type=int, default=None, help="per data-parallel rank")
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--no-sp", action="store_true", help="tp mode without sequence parallelism")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--microbatches", type=int, default=4)
    ap.add_argument("--no-symm", action="store_true", help="plain NCCL collectives instead of peer-memory kernels")
    ap.add_argument("--mode-steps", type=int, default=30, help="timed steps of each entry under 'modes'")
    ap.add_argument("--no-modes", action="store_true", help="headline only")
    ap.add_argument("--bucket-mb", type=float, default=25.0, help="gradient bucket size of the data-parallel wrapper")
    ap.add_argument("--modes-budget-s", type=float, default=240.0,
                    help="no further entry under 'modes' is started once the run is this old (wall clock of rank 0); "
                         "the headline is always measured")
    args = ap.parse_args()
    args.explicit_mode = args.mode is not None
    if args.mode is None:
        args.mode = "dp"
    return args


# --------------------------------------------------------------- clock sampler --
class ClockSampler:
    """Samples SM clock and throttle reasons of this rank's GPU while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# -------------------------------------------------------------------- helpers --
def model_knobs(name: str, seq: int, mode: str, knobs: str = "gpt2") -> dict:
    sizes = {"345m": (24, 1024, 16), "760m": (24, 1536, 16), "1.3b": (24, 2048, 16), "small": (4, 256, 4)}
    layers, hidden, heads = sizes[name]
    base = dict(max_seq_len=seq, hidden_size=hidden, num_layers=layers, num_heads=heads,
                ffn_hidden_size=4 * hidden, use_fused_qkv=True, attn_backend="flash")
    if knobs == "published":
        # nano_megatron scripts/benchmark_tp.py:94-113
        return dict(base, vocab_size=51200 if name != "small" else 1024, use_bias=False, tie_word_embeddings=False,
                    position_embedding_type="rope", activation_func="swiglu", gated_linear_unit=True)
    return dict(base, vocab_size=50304 if name != "small" else 1024, use_bias=True,
                tie_word_embeddings=(mode != "pp"), position_embedding_type="learned_absolute",
                activation_func="gelu", gated_linear_unit=False)


def layout(args) -> dict:
    n = args.gpus
    if args.mode == "dp" or n == 1:
        return dict(tp=1, cp=1, pp=1, dp=n, sp=False, name=f"dp{n}")
    if args.mode == "tp":
        return dict(tp=n, cp=1, pp=1, dp=1, sp=not args.no_sp, name=f"tp{n}" + ("" if args.no_sp else "+sp"))
    if args.mode == "cp":
        return dict(tp=1, cp=n, pp=1, dp=1, sp=False, name=f"cp{n}")
    if n == 8:
        return dict(tp=2, cp=1, pp=2, dp=2, sp=False, name="tp2xpp2xdp2")
    if n == 4:
        return dict(tp=2, cp=1, pp=2, dp=1, sp=False, name="tp2xpp2")
    return dict(tp=1, cp=1, pp=2, dp=1, sp=False, name="pp2")


def spec_of(args) -> dict:
    """Workload of one configuration: layout, model knobs, batch and sequence."""
    lay = layout(args)
    multi_pp = args.mode == "pp" and args.gpus > 1
    seq = args.seq or (1024 if multi_pp else 2048)
    if args.mode == "cp" and args.gpus > 1 and args.seq is None:
        seq = 2048 * args.gpus  # per-rank 2048 tokens, as the reference scales CP
    batch = args.batch or (8 if multi_pp else (1 if args.model == "1.3b" else 2))
    knobs = model_knobs(args.model, seq, args.mode if args.gpus > 1 else "dp", args.knobs)
    return dict(lay=lay, knobs=knobs, batch=batch, seq=seq, mode=args.mode, model=args.model,
                knob_set=args.knobs, microbatches=args.microbatches)


def extra_specs(args) -> list[tuple[str, argparse.Namespace]]:
    """The other configurations of the suite at this GPU count."""
    def variant(**kw) -> argparse.Namespace:
        ns = argparse.Namespace(**vars(args))
        ns.batch = ns.seq = None
        for k, v in kw.items():
            setattr(ns, k, v)
        return ns

    n = args.gpus
    out = [(f"dp{n}-760m", variant(mode="dp", model="760m"))]
    if n == 1:
        out.append(("1gpu-1.3b", variant(mode="dp", model="1.3b")))
    else:
        out.append((f"tp{n}+sp-345m", variant(mode="tp", model="345m")))
        out.append((f"cp{n}-1.3b", variant(mode="cp", model="1.3b")))
    if n in (2, 4, 8):
        out.append((layout(variant(mode="pp"))["name"] + "-345m", variant(mode="pp", model="345m")))
    out.append((f"dp{n}-345m-published-knobs", variant(mode="dp", model="345m", knobs="published")))
    return out


def init_normal(model, std: float = 0.02) -> None:
    import torch
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() > 1:
                p.normal_(0.0, std)
            elif name.endswith("bias"):
                p.zero_()


def describe(spec: dict) -> str:
    k = spec["knobs"]
    style = ("RoPE, SwiGLU, no bias, fused QKV" if spec["knob_set"] == "published"
             else "GELU, learned positions, bias, fused QKV")
    return (f"GPT-{spec['model']} (L{k['num_layers']} H{k['hidden_size']} h{k['num_heads']} F{k['ffn_hidden_size']} "
            f"V{k['vocab_size']}, {style}" + (", tied" if k["tie_word_embeddings"] else ", untied") + ")")


def emit(payload: dict) -> None:
    print(json.dumps(payload), flush=True)


# ------------------------------------------------------------------ measuring --
def measure(args, spec: dict, steps: int, warmup: int) -> dict:
    """Build one configuration, time it three ways, tear it down."""
    import torch
    import torch.distributed as dist

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    lay, knobs, batch, seq = spec["lay"], spec["knobs"], spec["batch"], spec["seq"]
    runner = (ReferenceRunner if args.impl == "reference" else B200Runner)(args, spec)
    torch.cuda.reset_peak_memory_stats(device)
    runner.build()

    gen = torch.Generator().manual_seed(1000 + runner.dp_rank)
    pool = [torch.randint(0, knobs["vocab_size"], (batch, seq), generator=gen).pin_memory() for _ in range(4)]
    ids_dev = [p.to(device) for p in pool]

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n: int, sample_clocks: bool = False):
        sampler = ClockSampler(local_rank) if sample_clocks else None
        if sampler is not None:
            sampler.start()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        last = None
        for i in range(n):
            last = fn(i)
        end.record()
        barrier()
        t = torch.tensor([start.elapsed_time(end)], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item(), last, (sampler.stop() if sampler is not None else None)

    # Set-up, not warm-up: the trainer runs a few eager steps and then captures
    # the step into a CUDA graph; do that before the W warm-up steps so that the
    # timed region never contains the capture, whatever W is.
    runner.prepare(ids_dev[0])
    barrier()

    # ---- device-timed region: inputs already resident ----
    for i in range(warmup):
        runner.step_device(ids_dev[i % 4])
    launches0 = runner.launch_counter()
    ms, loss, clocks = timed(lambda i: runner.step_device(ids_dev[i % 4]), steps, sample_clocks=True)
    per_step_launches = runner.launches_per_step(runner.launch_counter() - launches0, steps)
    final_loss = float(loss.item()) if loss is not None else None

    # ---- end to end: pinned host inputs in, loss out, every step ----
    for i in range(2):
        runner.step_host(pool[i % 4])
    ms_e2e, _, _ = timed(lambda i: runner.step_host(pool[i % 4]), steps)

    # ---- the reference's benchmark step: no optimizer update ----
    runner.prepare_no_optimizer(ids_dev[0])   # set-up (eager steps + capture), as above
    barrier()
    for i in range(max(warmup, 3)):
        runner.step_no_optimizer(ids_dev[i % 4])
    ms_nopt, _, _ = timed(lambda i: runner.step_no_optimizer(ids_dev[i % 4]), steps)
    runner.check()

    peak = torch.tensor([torch.cuda.max_memory_allocated(device) + runner.extra_device_bytes()],
                        dtype=torch.float64, device=device)
    dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    tokens_per_step = batch * seq * lay["dp"]
    out = {
        "tokens_per_step": tokens_per_step,
        "value": tokens_per_step * steps / (ms / 1e3), "ms_per_step": ms / steps,
        "e2e_value": tokens_per_step * steps / (ms_e2e / 1e3), "e2e_ms_per_step": ms_e2e / steps,
        "nopt_value": tokens_per_step * steps / (ms_nopt / 1e3), "nopt_ms_per_step": ms_nopt / steps,
        "peak_mem_mb": peak.item() / 2 ** 20, "clocks": clocks, "loss": final_loss,
        "launches_per_step": per_step_launches, "graphed": runner.graphed, "note": runner.note,
        "h2d": int(pool[0].numel() * pool[0].element_size()),
    }
    barrier()
    runner.close()
    del runner, pool, ids_dev
    gc.collect()
    torch.cuda.empty_cache()
    barrier()
    return out


def mode_entry(spec: dict, m: dict, steps: int) -> dict:
    return {
        "config": {"model": describe(spec), "global_batch": spec["batch"] * spec["lay"]["dp"],
                   "per_rank_batch": spec["batch"], "seq_len": spec["seq"], "parallelism": spec["lay"]["name"]},
        "value": round(m["value"], 1), "unit": "tokens/s", "ms_per_step": round(m["ms_per_step"], 3), "steps": steps,
        "e2e": {"value": round(m["e2e_value"], 1), "ms_per_step": round(m["e2e_ms_per_step"], 3)},
        "step_without_optimizer": {"value": round(m["nopt_value"], 1), "unit": "tokens/s",
                                   "ms_per_step": round(m["nopt_ms_per_step"], 3)},
        "peak_mem_mb": round(m["peak_mem_mb"], 1), "loss": m["loss"],
        **({"note": m["note"]} if m["note"] else {}),
    }


# ------------------------------------------------------------------------ main --
def main() -> int:
    args = parse_args()
    if args.impl == "nccl-baseline":
        args.no_symm = True
    if args.mode == "composite":
        args.mode = "pp"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # Convenience: re-launch under torchrun.
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", "29577", os.path.abspath(__file__), *sys.argv[1:]]
            return subprocess.call(cmd)
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")

    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "nano_megatron")):
        if rank == 0:
            emit({"impl": "reference", "unavailable": "baseline/_ref/nano_megatron is not installed"})
        return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        if rank == 0:
            emit({"impl": args.impl, "unavailable": "no CUDA device"})
        return 0
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29578")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    # One process group for the whole run; every configuration builds its
    # parallel context (and its sub-groups) on top of it and tears it down again.
    import datetime
    dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank),
                            timeout=datetime.timedelta(seconds=600))

    spec = spec_of(args)
    head = measure(args, spec, args.steps, args.warmup)

    modes: dict[str, dict] = {}
    if not args.explicit_mode and not args.no_modes:
        sub_steps = max(1, min(args.mode_steps, args.steps))
        for name, ns in extra_specs(args):
            sub = spec_of(ns)
            # Every configuration costs tens of seconds of set-up (groups, workspaces, capture):
            # stop adding entries when the run is older than the budget.  Rank 0's clock decides.
            age = torch.tensor([time.time() - T_START], device=torch.device("cuda", local_rank))
            dist.broadcast(age, src=0)
            if age.item() > args.modes_budget_s:
                modes[name] = {"skipped": f"time budget of {args.modes_budget_s:.0f} s for the sub-results was used up"}
                continue
            try:
                modes[name] = mode_entry(sub, measure(ns, sub, sub_steps, max(3, min(args.warmup, 5))), sub_steps)
            except Exception as exc:  # one configuration must not cost the whole line
                modes[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
                # the ranks may have diverged: no further collective configuration is safe
                break

    lay, knobs = spec["lay"], spec["knobs"]
    published = PUBLISHED.get((args.model, args.mode, args.gpus)) if args.knobs == "gpt2" else None
    if rank == 0:
        out = {
            "metric": METRIC,
            "value": round(head["value"], 1), "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(head["ms_per_step"], 3), "higher_is_better": True,
            "scaling": "weak" if args.mode in ("dp", "cp") else "strong",
            "vs_baseline": round(head["value"] / published, 3) if published else None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init normal(0,0.02) weights",
            "impl": args.impl,
            "config": {"model": describe(spec),
                       "global_batch": spec["batch"] * lay["dp"], "per_rank_batch": spec["batch"],
                       "seq_len": spec["seq"], "parallelism": lay["name"], "optimizer": "AdamW in the timed region",
                       "attention": "flash",
                       "l2": "working set (weights + activations, > 2 GB) exceeds the 126 MB L2; no flush needed",
                       "vs_baseline_note": "published number is the reference on 4x RTX A6000 without optimizer step"
                       if published else "no published number for this configuration"},
            "clocks": head["clocks"],
            "e2e": {"value": round(head["e2e_value"], 1), "unit": "tokens/s",
                    "ms_per_step": round(head["e2e_ms_per_step"], 3),
                    "h2d_bytes_per_step": head["h2d"], "d2h_bytes_per_step": 4},
            "step_without_optimizer": {"value": round(head["nopt_value"], 1), "unit": "tokens/s",
                                       "ms_per_step": round(head["nopt_ms_per_step"], 3),
                                       "what": "zero-grad, forward, loss, backward, gradient sync (the reference's "
                                               "own benchmark step)"},
            "peak_mem_mb": round(head["peak_mem_mb"], 1),
            "gpu_launches": int(head["launches_per_step"] * args.steps),
            "cuda_graph": head["graphed"],
            "loss": head["loss"],
        }
        if modes:
            out["modes"] = modes
        if head["note"]:
            out["note"] = head["note"]
        emit(out)

    # The result is out.  Tear down in order and leave through the normal
    # interpreter exit (exit handlers run).  A timer stands by only in case
    # communicator destruction stalls: then it ends the process.
    sys.stdout.flush()
    sys.stderr.flush()
    fallback = _arm_exit_timer(90.0)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    fallback.cancel()
    return 0


def _arm_exit_timer(seconds: float) -> threading.Timer:
    def fire() -> None:
        sys.stderr.write("bench.py: teardown did not finish in time; leaving\n")
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)

    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()
    return t


class B200Runner:
    """This framework through its public API (``Trainer`` / ``PipelineTrainer``)."""

    def __init__(self, args, spec) -> None:
        self.args, self.spec = args, spec
        self.lay, self.knobs, self.batch, self.seq = spec["lay"], spec["knobs"], spec["batch"], spec["seq"]
        self.note = None
        self.graphed = False

    def build(self) -> None:
        import torch
        import nano_megatron_b200.parallel as P
        from nano_megatron_b200.engine import Trainer
        from nano_megatron_b200.models import build_pipeline_stage_from_reference, build_tp_gpt_from_reference
        from nano_megatron_b200.reference import ReferenceGPT, ReferenceGPTConfig, seed_all

        lay = self.lay
        self.P = P
        self.ctx = P.initialize_parallel(P.ParallelConfig(
            tensor_parallel_size=lay["tp"], context_parallel_size=lay["cp"], pipeline_parallel_size=lay["pp"],
            sequence_parallel=lay["sp"]), dist_backend="nccl")
        self.dp_rank = self.ctx.data_parallel_rank
        self.workspaces = {}
        if not self.args.no_symm and self.ctx.world_size > 1:
            try:
                from nano_megatron_b200.distributed.symm_mem import enable_symmetric_memory
                self.workspaces = enable_symmetric_memory(self.ctx)
            except Exception as exc:  # plain NCCL stays available
                self.note = f"symmetric memory unavailable ({type(exc).__name__}: {exc}); NCCL collectives used"
        seed_all(42)
        cfg = ReferenceGPTConfig(**self.knobs)
        dev = torch.device("cuda", self.ctx.local_rank)
        with torch.device(dev):
            ref = ReferenceGPT(cfg)
        init_normal(ref)
        if lay["pp"] > 1:
            from nano_megatron_b200.engine import PipelineTrainer
            stage = build_pipeline_stage_from_reference(ref, self.ctx).to(dev, dtype=torch.bfloat16)
            self.trainer = PipelineTrainer(stage, self.ctx, num_microbatches=self.spec["microbatches"], lr=1e-4,
                                           weight_decay=0.01, use_cuda_graph=not self.args.no_graph)
        else:
            model = build_tp_gpt_from_reference(ref, self.ctx).to(dev, dtype=torch.bfloat16)
            self.trainer = Trainer(model, self.ctx, lr=1e-4, weight_decay=0.01, bucket_cap_mb=self.args.bucket_mb,
                                   use_cuda_graph=not self.args.no_graph)
        del ref

    def step_device(self, ids_dev):
        loss = self.trainer.step(ids_dev)
        self.graphed = self.trainer.graphed
        return loss

    def step_no_optimizer(self, ids_dev):
        return self.trainer.forward_backward(ids_dev)

    def prepare(self, ids_dev) -> None:
        for _ in range(6):
            if self.trainer.graphed or self.trainer.graph_error or self.args.no_graph:
                break
            self.trainer.step(ids_dev)
        self.graphed = self.trainer.graphed

    def prepare_no_optimizer(self, ids_dev) -> None:
        settled = getattr(self.trainer, "graph_settled", None)
        for _ in range(8):
            if settled is None or self.args.no_graph or settled(False):
                break
            self.trainer.forward_backward(ids_dev)

    def step_host(self, ids_pinned):
        loss = self.trainer.step(ids_pinned)
        return None if loss is None else loss.item()

    def launch_counter(self) -> int:
        from nano_megatron_b200.ops import native
        return native.launches

    def launches_per_step(self, counted: int, steps: int) -> float:
        if self.trainer.graphed:
            return float(self.trainer.kernels_in_graph)
        return counted / max(steps, 1)

    def extra_device_bytes(self) -> int:
        return sum(ws.allocated_bytes() for ws in self.workspaces.values())

    def check(self) -> None:
        from nano_megatron_b200.ops import native
        native.check_status()
        if self.trainer.graph_error and self.note is None:
            self.note = f"not every step kind runs from a CUDA graph: {self.trainer.graph_error}"

    def close(self) -> None:
        if self.trainer is not None:
            self.trainer.close()        # graphs and gradient hooks would keep the model alive
        self.trainer = None
        self.P.destroy_parallel()


class ReferenceRunner:
    """The unmodified reference package: its models, DDP, schedule and AdamW."""

    def __init__(self, args, spec) -> None:
        self.args, self.spec = args, spec
        self.lay, self.knobs, self.batch, self.seq = spec["lay"], spec["knobs"], spec["batch"], spec["seq"]
        self.note = None
        self.graphed = False

    def build(self) -> None:
        import torch
        from nano_megatron.distributed.ddp import DistributedDataParallel
        from nano_megatron.model import build_pipeline_stage_from_reference, build_tp_gpt_from_reference
        from nano_megatron.parallel import ParallelConfig, destroy_parallel, initialize_parallel
        from nano_megatron.reference import AdamW, ReferenceGPT, ReferenceGPTConfig
        from nano_megatron.reference.loss import shifted_cross_entropy

        lay = self.lay
        self._destroy = destroy_parallel
        self.ctx = initialize_parallel(ParallelConfig(
            tensor_parallel_size=lay["tp"], context_parallel_size=lay["cp"], pipeline_parallel_size=lay["pp"],
            sequence_parallel=lay["sp"]), dist_backend="nccl")
        self.dp_rank = self.ctx.data_parallel_rank
        torch.manual_seed(42)
        torch.cuda.manual_seed_all(42)
        cfg = ReferenceGPTConfig(**self.knobs)
        dev = torch.device("cuda", self.ctx.local_rank)
        with torch.device(dev):
            ref = ReferenceGPT(cfg)
        init_normal(ref)
        self.dev = dev
        if lay["pp"] > 1:
            self.stage = build_pipeline_stage_from_reference(ref, self.ctx).to(dev, dtype=torch.bfloat16)
            self.module = self.stage
        elif lay["tp"] > 1 or lay["cp"] > 1:
            self.module = build_tp_gpt_from_reference(ref, self.ctx).to(dev, dtype=torch.bfloat16)
        else:
            self.module = ref.to(dev, dtype=torch.bfloat16)
        self.ddp = DistributedDataParallel(self.module, self.ctx)
        self.opt = AdamW(self.module.named_parameters(), lr=1e-4, weight_decay=0.01)
        self._plain_ce = shifted_cross_entropy

    def _forward_backward(self, ids):
        if self.lay["pp"] > 1:
            from nano_megatron.schedules import forward_backward_1f1b
            return forward_backward_1f1b(stage=self.stage, ctx=self.ctx, input_ids=ids, labels=ids,
                                         num_microbatches=self.spec["microbatches"], ddp=self.ddp)
        logits = self.ddp(ids)
        if hasattr(self.module, "shifted_cross_entropy"):
            loss = self.module.shifted_cross_entropy(logits, ids)
        else:
            loss = self._plain_ce(logits, ids)
        loss.backward()
        self.ddp.finish_grad_sync()
        return loss

    def _step(self, ids):
        loss = self._forward_backward(ids)
        self.opt.step()
        self.ddp.zero_grad(set_to_none=True)
        return loss

    def step_device(self, ids_dev):
        return self._step(ids_dev)

    def step_no_optimizer(self, ids_dev):
        # the loop of the reference's own benchmark scripts (scripts/benchmark_dp.py:212-223)
        loss = self._forward_backward(ids_dev)
        self.ddp.zero_grad(set_to_none=True)
        return loss

    def step_host(self, ids_pinned):
        loss = self._step(ids_pinned.to(self.dev, non_blocking=True))
        return None if loss is None else loss.item()

    def launch_counter(self) -> int:
        return 0

    def launches_per_step(self, counted: int, steps: int) -> float:
        return 0.0

    def extra_device_bytes(self) -> int:
        return 0

    def check(self) -> None:
        pass

    def prepare(self, ids_dev) -> None:
        pass

    def prepare_no_optimizer(self, ids_dev) -> None:
        pass

    def close(self) -> None:
        self.opt = self.ddp = self.module = self.stage = None
        self._destroy()


if __name__ == "__main__":
    sys.exit(main())
