"""Throughput / roofline bookkeeping and JSON-lines logging.

The reference prints on rank 0 and fills ``BenchmarkResult`` dataclasses
(scripts/benchmark_tp.py:149-159,402-487).  Here the same three metrics
(tokens/s, peak memory, step time) plus model FLOPs and the fraction of the
measured machine peak are produced as dictionaries and appended to a
JSON-lines file."""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Optional

import torch


@dataclass
class StepMetrics:
    step: int
    loss: float
    ms: float
    tokens: int
    tokens_per_s: float
    peak_mem_mb: float = 0.0
    extra: dict[str, Any] = field(default_factory=dict)


def gpt_train_flops(num_layers: int, hidden: int, ffn: int, vocab: int, seq: int, tokens: int,
                    gated: bool = False) -> float:
    """Forward + backward matmul FLOPs of one step (attention counted causal)."""
    per_token_layer = 2 * (3 * hidden * hidden + hidden * hidden + (3 if gated else 2) * hidden * ffn)
    attn = 2 * 2 * seq * hidden / 2          # QK^T and PV, half masked
    fwd = tokens * (num_layers * (per_token_layer + attn) + 2 * hidden * vocab)
    return 3.0 * fwd


def measured_peaks(path: Optional[str] = None) -> dict[str, float]:
    """Roofline denominators: the driver-measured file when present, else the
    documented fallback of an earlier measurement on the same kind of GPU."""
    for cand in filter(None, (path, os.environ.get("NMB_MEASURED_PEAKS"),
                              os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(__file__))),
                                           "MEASURED_PEAKS.json"))):
        if os.path.exists(cand):
            with open(cand) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def roofline_fraction(flops: float, bytes_moved: float, seconds: float, peaks: Optional[dict] = None) -> dict[str, float]:
    peaks = peaks or measured_peaks()
    t_compute = flops / (peaks["bf16_tflops"] * 1e12)
    t_memory = bytes_moved / (peaks["hbm_gbs"] * 1e9)
    bound = max(t_compute, t_memory)
    return {"achieved_tflops": flops / seconds / 1e12, "achieved_gbs": bytes_moved / seconds / 1e9,
            "roofline_s": bound, "fraction": bound / seconds if seconds > 0 else 0.0,
            "bound": "compute" if t_compute >= t_memory else "memory", "peaks": peaks["source"]}


class JsonlLogger:
    """Rank-0 JSON-lines writer (one object per call)."""

    def __init__(self, path: str, rank: int = 0) -> None:
        self.path, self.rank = path, rank
        if rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def log(self, record: Any) -> None:
        if self.rank != 0:
            return
        if hasattr(record, "__dataclass_fields__"):
            record = asdict(record)
        record = dict(record)
        record.setdefault("time", time.time())
        with open(self.path, "a") as f:
            f.write(json.dumps(record) + "\n")


def peak_memory_mb(device: Optional[torch.device] = None) -> float:
    if not torch.cuda.is_available():
        return 0.0
    return torch.cuda.max_memory_allocated(device) / (1024 * 1024)
