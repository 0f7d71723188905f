"""The parts of the benchmark contract that can be checked without a GPU:
defaults, layouts per mode and GPU count, the model shapes behind the preset
names, the clock-sample parser and the no-device answers."""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def _args(**kw):
    base = dict(gpus=1, mode="dp", no_sp=False)
    base.update(kw)
    return argparse.Namespace(**base)


def test_defaults_are_one_gpu_and_enough_warmup(monkeypatch):
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    a = bench.parse_args()
    assert a.gpus == 1 and a.steps >= 1 and a.warmup >= 3 and a.impl == "b200" and a.mode == "dp" and a.model == "345m"


@pytest.mark.parametrize("mode,n,want", [
    ("dp", 1, dict(dp=1, tp=1, cp=1, pp=1)), ("dp", 8, dict(dp=8, tp=1, cp=1, pp=1)),
    ("tp", 1, dict(dp=1, tp=1, cp=1, pp=1)),                     # one GPU is always the plain layout
    ("tp", 4, dict(dp=1, tp=4, cp=1, pp=1, sp=True)), ("cp", 2, dict(dp=1, tp=1, cp=2, pp=1)),
    ("pp", 2, dict(dp=1, tp=1, cp=1, pp=2)), ("pp", 4, dict(dp=1, tp=2, cp=1, pp=2)),
    ("pp", 8, dict(dp=2, tp=2, cp=1, pp=2)),
])
def test_layouts_fill_exactly_the_requested_gpus(mode, n, want):
    lay = bench.layout(_args(gpus=n, mode=mode))
    assert lay["tp"] * lay["cp"] * lay["pp"] * lay["dp"] == n
    for k, v in want.items():
        assert lay[k] == v, (k, lay)
    import nano_megatron_b200.parallel as P
    P.ParallelConfig(tensor_parallel_size=lay["tp"], context_parallel_size=lay["cp"],
                     pipeline_parallel_size=lay["pp"], sequence_parallel=lay["sp"]).validate(n)


def test_tp_mode_can_drop_sequence_parallelism():
    assert bench.layout(_args(gpus=2, mode="tp", no_sp=True))["sp"] is False


@pytest.mark.parametrize("name,params_m", [("345m", 355.9), ("760m", 760.4), ("1.3b", 1315.8)])
def test_preset_shapes_are_the_gpt2_style_models_of_the_baseline(name, params_m):
    import torch

    from nano_megatron_b200.reference import ReferenceGPT, ReferenceGPTConfig

    knobs = bench.model_knobs(name, 2048, "dp")
    assert knobs["vocab_size"] == 50304 and knobs["num_layers"] == 24 and knobs["ffn_hidden_size"] == 4 * knobs["hidden_size"]
    assert knobs["tie_word_embeddings"] and not bench.model_knobs(name, 1024, "pp")["tie_word_embeddings"]
    with torch.device("meta"):
        model = ReferenceGPT(ReferenceGPTConfig(**{**knobs, "attn_backend": "unfused"}))
    seen, total = set(), 0
    for p in model.parameters():
        if id(p) not in seen:
            seen.add(id(p))
            total += p.numel()
    assert total / 1e6 == pytest.approx(params_m, abs=0.1)


def test_clock_sample_parser(monkeypatch):
    sampler = bench.ClockSampler(0)

    class _Proc:
        def terminate(self):
            pass

        def communicate(self, timeout=None):
            return ("1965, 1965, 412.3, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active\n"
                    "1500, 1965, 998.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
                    "garbage line\n"
                    "1600, 1965, 990.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"), None

    sampler.proc = _Proc()
    got = sampler.stop()
    assert got == {"sm_mhz": 1600.0, "sm_max_mhz": 1965.0, "samples": 3, "reasons": ["sw_power_cap"]}
    assert bench.ClockSampler(0).stop()["reasons"] == ["nvidia-smi unavailable"]


@pytest.mark.parametrize("impl", ["b200", "reference"])
def test_without_a_device_one_json_line_says_so_and_the_exit_code_is_zero(impl):
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    env["CUDA_VISIBLE_DEVICES"] = ""
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", impl, "--steps", "1", "--warmup", "1"],
                          capture_output=True, text=True, timeout=120, env=env)
    assert proc.returncode == 0, proc.stderr[-500:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    payload = json.loads(lines[0])
    assert payload["impl"] == impl and "unavailable" in payload
