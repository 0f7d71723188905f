#!/usr/bin/env python
"""Headline benchmark: GPT training tokens/sec on N GPUs of one node.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W [--mode dp|tp|cp|pp] [--impl reference]

One step = zero-grad, forward, shifted cross entropy, backward, gradient
synchronisation and an AdamW update, bf16 parameters, synthetic uniform token
ids, random-init weights.  Rank 0 prints ONE JSON line.

``--impl reference`` runs the unmodified reference package (installed offline
into ``baseline/_ref``) through its own modules for the same step and config.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

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


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "nccl-baseline", "reference"],
                    help="b200: this framework; nccl-baseline: this framework's modules on plain NCCL collectives "
                         "(same as --no-symm); reference: the unmodified reference package")
    ap.add_argument("--mode", default="dp", choices=["dp", "tp", "cp", "pp", "composite"],
                    help="composite = pp: TP2 x PP2 (x DP2 at 8 GPUs) with the 1F1B schedule")
    ap.add_argument("--model", default="345m", choices=["345m", "760m", "1.3b", "small"])
    ap.add_argument("--batch", type=int, default=None, help="per data-parallel rank")
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--no-sp", action="store_true", help="tp mode without sequence parallelism")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--microbatches", type=int, default=4)
    ap.add_argument("--no-symm", action="store_true", help="plain NCCL collectives instead of peer-memory kernels")
    return ap.parse_args()


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
def model_knobs(name: str, seq: int, mode: str) -> dict:
    sizes = {"345m": (24, 1024, 16), "760m": (24, 1536, 16), "1.3b": (24, 2048, 16), "small": (4, 256, 4)}
    layers, hidden, heads = sizes[name]
    return dict(vocab_size=50304 if name != "small" else 1024, max_seq_len=seq, hidden_size=hidden,
                num_layers=layers, num_heads=heads, ffn_hidden_size=4 * hidden, use_bias=True,
                tie_word_embeddings=(mode != "pp"), position_embedding_type="learned_absolute",
                activation_func="gelu", gated_linear_unit=False, use_fused_qkv=True, attn_backend="flash")


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


def init_normal(model, std: float = 0.02) -> None:
    import torch
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() > 1:
                p.normal_(0.0, std)
            elif name.endswith("bias"):
                p.zero_()


def emit(payload: dict) -> None:
    print(json.dumps(payload), flush=True)


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

    lay = layout(args)
    seq = args.seq or (1024 if args.mode == "pp" and args.gpus > 1 else 2048)
    if args.mode == "cp" and args.gpus > 1 and args.seq is None:
        seq = 2048 * args.gpus  # per-rank 2048 tokens, as the reference scales CP
    batch = args.batch or (8 if args.mode == "pp" and args.gpus > 1 else (1 if args.model == "1.3b" else 2))
    knobs = model_knobs(args.model, seq, args.mode if args.gpus > 1 else "dp")

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        runner = ReferenceRunner(args, lay, knobs, batch, seq)
    else:
        runner = B200Runner(args, lay, knobs, batch, seq)
    runner.build()

    device = torch.device("cuda", local_rank)
    dp_rank = runner.dp_rank
    gen = torch.Generator().manual_seed(1000 + dp_rank)
    pool = [torch.randint(0, knobs["vocab_size"], (batch, seq), generator=gen).pin_memory() for _ in range(4)]
    ids_dev = [p.to(device) for p in pool]

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    # Set-up, not warm-up: the trainer runs a few eager steps and then captures
    # the step into a CUDA graph; do that before the W warm-up steps so that the
    # timed region never contains the capture, whatever W is.
    runner.prepare(ids_dev[0])
    barrier()

    # ---- device-timed region: inputs already resident ----
    for i in range(args.warmup):
        runner.step_device(ids_dev[i % 4])
    barrier()
    from nano_megatron_b200.ops import native as _native
    launches0 = _native.launches
    sampler = ClockSampler(local_rank)
    sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(args.steps):
        loss = runner.step_device(ids_dev[i % 4])
    end.record()
    barrier()
    ms = start.elapsed_time(end)
    clocks = sampler.stop()
    per_step_launches = runner.launches_per_step(_native.launches - launches0, args.steps)
    t = torch.tensor([ms], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    final_loss = float(loss.item()) if loss is not None else None

    # ---- end to end: pinned host inputs in, loss out, every step ----
    for i in range(2):
        runner.step_host(pool[i % 4])
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for i in range(args.steps):
        runner.step_host(pool[i % 4])
    e2.record()
    barrier()
    t2 = torch.tensor([s2.elapsed_time(e2)], device=device)
    dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    ms_e2e = t2.item()
    runner.check()

    tokens_per_step = batch * seq * lay["dp"]
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (ms_e2e / 1e3)
    published = PUBLISHED.get((args.model, args.mode, args.gpus))
    if rank == 0:
        out = {
            "metric": "training tokens/sec/box (device-timed, max over ranks), fwd+bwd+grad-sync+AdamW, bf16",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
            "scaling": "weak" if args.mode in ("dp", "cp") else "strong",
            "vs_baseline": round(value / published, 3) if published else None,
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init normal(0,0.02) weights",
            "impl": args.impl,
            "config": {"model": f"GPT-{args.model} (L{knobs['num_layers']} H{knobs['hidden_size']} "
                                f"h{knobs['num_heads']} F{knobs['ffn_hidden_size']} V{knobs['vocab_size']}, GELU, "
                                "learned positions, bias, fused QKV" + (", tied" if knobs["tie_word_embeddings"] else ", untied") + ")",
                       "global_batch": batch * lay["dp"], "per_rank_batch": batch, "seq_len": seq,
                       "parallelism": lay["name"], "optimizer": "AdamW in the timed region",
                       "attention": "flash", "cuda_graph": runner.graphed,
                       "l2": "working set (weights + activations, > 2 GB) exceeds the 126 MB L2; no flush needed",
                       "vs_baseline_note": "published number is the reference on 4x RTX A6000 without optimizer step"
                       if published else "no published number for this configuration"},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e / args.steps, 3),
                    "h2d_bytes_per_step": int(pool[0].numel() * pool[0].element_size()), "d2h_bytes_per_step": 4},
            "gpu_launches": int(per_step_launches * args.steps),
            "loss": final_loss,
        }
        if runner.note:
            out["note"] = runner.note
        emit(out)
    # The result is out.  Tear down in order, but never let teardown (NCCL
    # communicator destruction, unmapping peer memory, interpreter finalisers)
    # hold the job: a timer ends the process if close() stalls, and the process
    # leaves without running finalisers once close() has returned.
    barrier()
    _arm_exit_timer(60.0)
    runner.close()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def _arm_exit_timer(seconds: float) -> None:
    import threading

    def fire() -> None:
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)

    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()


class B200Runner:
    """This framework through its public API (``Trainer`` / ``forward_backward_1f1b``)."""

    def __init__(self, args, lay, knobs, batch, seq) -> None:
        self.args, self.lay, self.knobs, self.batch, self.seq = args, lay, knobs, batch, seq
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
        if not self.args.no_symm and self.ctx.world_size > 1:
            try:
                from nano_megatron_b200.distributed.symm_mem import enable_symmetric_memory
                enable_symmetric_memory(self.ctx)
            except Exception as exc:  # plain NCCL stays available
                self.note = f"symmetric memory unavailable ({type(exc).__name__}: {exc}); NCCL collectives used"
        seed_all(42)
        cfg = ReferenceGPTConfig(**self.knobs)
        with torch.device("cpu"):
            ref = ReferenceGPT(cfg)
        init_normal(ref)
        dev = torch.device("cuda", self.ctx.local_rank)
        if lay["pp"] > 1:
            from nano_megatron_b200.distributed import DistributedDataParallel
            from nano_megatron_b200.reference import AdamW
            self.stage = build_pipeline_stage_from_reference(ref, self.ctx).to(dev, dtype=torch.bfloat16)
            self.ddp = DistributedDataParallel(self.stage, self.ctx)
            self.opt = AdamW(self.stage.named_parameters(), lr=1e-4, weight_decay=0.01)
            self.trainer = None
        else:
            model = build_tp_gpt_from_reference(ref, self.ctx).to(dev, dtype=torch.bfloat16)
            self.trainer = Trainer(model, self.ctx, lr=1e-4, weight_decay=0.01,
                                   use_cuda_graph=not self.args.no_graph)
        del ref
        self._ids_static = None

    def _pp_step(self, ids):
        from nano_megatron_b200.schedules import forward_backward_1f1b
        self.ddp.zero_grad()
        loss = forward_backward_1f1b(stage=self.stage, ctx=self.ctx, input_ids=ids, labels=ids,
                                     num_microbatches=self.args.microbatches, ddp=self.ddp)
        self.opt.step()
        return loss

    def step_device(self, ids_dev):
        if self.trainer is None:
            return self._pp_step(ids_dev)
        loss = self.trainer.step(ids_dev)
        self.graphed = self.trainer.graphed
        return loss

    def prepare(self, ids_dev) -> None:
        if self.trainer is None:
            return
        for _ in range(6):
            if self.trainer.graphed or self.trainer.graph_error or self.args.no_graph:
                break
            self.trainer.step(ids_dev)
        self.graphed = self.trainer.graphed

    def step_host(self, ids_pinned):
        import torch
        if self.trainer is None:
            loss = self._pp_step(ids_pinned.to(torch.device("cuda", self.ctx.local_rank), non_blocking=True))
            return None if loss is None else loss.item()
        return self.trainer.step(ids_pinned).item()

    def launches_per_step(self, counted: int, steps: int) -> float:
        if self.trainer is not None and self.trainer.graphed:
            return float(self.trainer.kernels_in_graph)
        return counted / max(steps, 1)

    def check(self) -> None:
        from nano_megatron_b200.ops import native
        native.check_status()
        if self.trainer is not None and self.trainer.graph_error and self.note is None:
            self.note = f"CUDA graph capture failed, eager launches used: {self.trainer.graph_error}"

    def close(self) -> None:
        self.P.destroy_parallel()


class ReferenceRunner:
    """The unmodified reference package: its models, DDP, schedule and AdamW."""

    def __init__(self, args, lay, knobs, batch, seq) -> None:
        self.args, self.lay, self.knobs, self.batch, self.seq = args, lay, knobs, batch, seq
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
        cfg = ReferenceGPTConfig(**self.knobs)
        ref = ReferenceGPT(cfg)
        init_normal(ref)
        dev = torch.device("cuda", self.ctx.local_rank)
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

    def _step(self, ids):
        if self.lay["pp"] > 1:
            from nano_megatron.schedules import forward_backward_1f1b
            loss = forward_backward_1f1b(stage=self.stage, ctx=self.ctx, input_ids=ids, labels=ids,
                                         num_microbatches=self.args.microbatches, ddp=self.ddp)
        else:
            logits = self.ddp(ids)
            if hasattr(self.module, "shifted_cross_entropy"):
                loss = self.module.shifted_cross_entropy(logits, ids)
            else:
                loss = self._plain_ce(logits, ids)
            loss.backward()
            self.ddp.finish_grad_sync()
        self.opt.step()
        self.ddp.zero_grad(set_to_none=True)
        return loss

    def step_device(self, ids_dev):
        return self._step(ids_dev)

    def step_host(self, ids_pinned):
        loss = self._step(ids_pinned.to(self.dev, non_blocking=True))
        return None if loss is None else loss.item()

    def launches_per_step(self, counted: int, steps: int) -> float:
        return 0.0

    def check(self) -> None:
        pass

    def prepare(self, ids_dev) -> None:
        pass

    def close(self) -> None:
        self._destroy()


if __name__ == "__main__":
    sys.exit(main())
