"""Checkpoint / resume, timers, metrics, watchdog and the oracle CLI (CPU)."""
from __future__ import annotations

import json
import os
import time

import pytest
import torch

import nano_megatron_b200.parallel as P
from nano_megatron_b200.models import build_tp_gpt_from_reference
from nano_megatron_b200.reference import AdamW, ReferenceGPT, ReferenceGPTConfig, seed_all
from nano_megatron_b200.utils import (
    CommTimeout,
    DeviceTimer,
    Heartbeat,
    JsonlLogger,
    StepMetrics,
    StepWatchdog,
    gpt_train_flops,
    load_checkpoint,
    measured_peaks,
    merge_checkpoint,
    roofline_fraction,
    save_checkpoint,
    shard_tensor,
    time_steps,
    unshard_tensor,
)
from tests._dist_utils import launch, port_for

HERE = os.path.abspath(__file__)


def _cfg(**kw):
    base = dict(num_layers=2, hidden_size=32, num_heads=4, vocab_size=64, max_seq_len=16, attn_backend="unfused",
                use_bias=True, use_fused_qkv=True)
    base.update(kw)
    return ReferenceGPTConfig(**base)


@pytest.fixture
def ctx(monkeypatch, request):
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", str(port_for(request.node.nodeid)))
    monkeypatch.setenv("RANK", "0")
    monkeypatch.setenv("WORLD_SIZE", "1")
    monkeypatch.delenv("LOCAL_RANK", raising=False)
    c = P.initialize_parallel(P.ParallelConfig(), dist_backend="gloo")
    yield c
    P.destroy_parallel()


def _train(model, opt, ids, steps):
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = model.shifted_cross_entropy(model(ids), ids)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses


def test_resume_reproduces_the_trajectory_bit_for_bit(ctx, tmp_path):
    seed_all(0)
    cfg = _cfg()
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    model = build_tp_gpt_from_reference(ReferenceGPT(cfg), ctx)
    opt = AdamW(model.named_parameters(), lr=1e-2, weight_decay=0.01)
    _train(model, opt, ids, 2)
    path = save_checkpoint(str(tmp_path), model, opt, ctx, step=2, extra={"note": "unit"})
    assert path and os.path.exists(path) and not os.path.exists(path + ".tmp")
    want = _train(model, opt, ids, 3)

    seed_all(99)                                              # a "new process": different init
    fresh = build_tp_gpt_from_reference(ReferenceGPT(cfg), ctx)
    fresh_opt = AdamW(fresh.named_parameters(), lr=1e-2, weight_decay=0.01)
    assert load_checkpoint(str(tmp_path), fresh, fresh_opt, ctx) == 2
    assert _train(fresh, fresh_opt, ids, 3) == want
    merged = merge_checkpoint(str(tmp_path))
    assert merged["extra"] == {"note": "unit"} and merged["optimizer"]["ln_f_weight"]["step"] == 2
    ref = ReferenceGPT(cfg)
    ref.load_state_dict(merged["model"])                      # loads into the oracle unchanged

    # the command-line merge writes the same thing as one portable file
    from nano_megatron_b200.cli import merge_checkpoint as merge_cli
    from nano_megatron_b200.reference import ReferenceGPTConfig
    out = str(tmp_path / "merged.pt")
    assert merge_cli.main([str(tmp_path), out]) == 0
    blob = torch.load(out, map_location="cpu", weights_only=False)
    again = ReferenceGPT(ReferenceGPTConfig(**blob["config"]))
    again.load_state_dict(blob["model"])
    assert blob["step"] == 2 and set(blob["optimizer"]) == set(merged["optimizer"])


@pytest.mark.parametrize("knobs", [dict(), dict(gated_linear_unit=True, num_query_groups=2)])
def test_shard_rules_round_trip(knobs):
    cfg = _cfg(**knobs)
    ref = ReferenceGPT(cfg)
    for name, p in ref.named_parameters():
        for tp in (2, 4):
            if name.endswith("k_proj.weight") and cfg.num_query_groups % tp:
                continue
            parts = [shard_tensor(name, p.data, cfg, r, tp) for r in range(tp)]
            assert torch.equal(unshard_tensor(name, parts, cfg), p.data), name


def worker_tp2_save():
    import torch.distributed as dist
    Pm = P
    ctx = Pm.initialize_parallel(Pm.ParallelConfig(tensor_parallel_size=2), dist_backend="gloo")
    seed_all(0)
    cfg = _cfg(gated_linear_unit=True)
    model = build_tp_gpt_from_reference(ReferenceGPT(cfg), ctx)
    opt = AdamW(model.named_parameters(), lr=1e-2)
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    _train(model, opt, ids, 2)
    save_checkpoint(os.environ["NMB_CKPT_DIR"], model, opt, ctx, step=2)
    nxt = _train(model, opt, ids, 1)[0]
    if ctx.rank == 0:
        with open(os.path.join(os.environ["NMB_CKPT_DIR"], "next_loss.json"), "w") as f:
            json.dump({"loss": nxt}, f)
    dist.barrier()
    Pm.destroy_parallel()


def test_tp2_checkpoint_reloads_at_tp1(ctx, tmp_path):
    launch(HERE, "worker_tp2_save", 2, timeout=180, extra_env={"NMB_CKPT_DIR": str(tmp_path)})
    assert sorted(os.listdir(tmp_path)) == ["next_loss.json", "shard_tp0_pp0.pt", "shard_tp1_pp0.pt"]
    cfg = _cfg(gated_linear_unit=True)
    seed_all(5)
    model = build_tp_gpt_from_reference(ReferenceGPT(cfg), ctx)
    opt = AdamW(model.named_parameters(), lr=1e-2)
    assert load_checkpoint(str(tmp_path), model, opt, ctx) == 2
    seed_all(0)
    ReferenceGPT(cfg)                                          # consume the same RNG as the worker did
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    got = _train(model, opt, ids, 1)[0]
    want = json.load(open(tmp_path / "next_loss.json"))["loss"]
    assert abs(got - want) < 1e-5 * max(1.0, abs(want))


def test_timers_and_step_timer():
    t = DeviceTimer(torch.device("cpu"))
    with t.region("a"):
        time.sleep(0.01)
    with t.region("a"):
        time.sleep(0.01)
    s = t.summary(reduce_max=False)
    assert s["a"] >= 15.0
    calls = []
    ms = time_steps(lambda: calls.append(1), warmup=2, steps=5)
    assert len(calls) == 7 and ms >= 0.0


def test_metrics_and_roofline(tmp_path):
    peaks = measured_peaks(path=str(tmp_path / "missing.json"))
    assert peaks["source"] in ("measured", "fallback") and peaks["hbm_gbs"] > 1000
    fl = gpt_train_flops(24, 1024, 4096, 50304, 2048, 4096)
    assert 8e12 < fl < 1.2e13                                 # ~6 * 355M params * 4096 tokens plus attention
    r = roofline_fraction(1e12, 1e9, 1e-3, {"hbm_gbs": 6500.0, "bf16_tflops": 1600.0, "source": "test"})
    assert r["bound"] == "compute" and abs(r["fraction"] - 0.625) < 1e-6
    log = JsonlLogger(str(tmp_path / "m" / "log.jsonl"))
    log.log(StepMetrics(step=1, loss=2.0, ms=3.0, tokens=4, tokens_per_s=5.0))
    rec = json.loads(open(tmp_path / "m" / "log.jsonl").read())
    assert rec["step"] == 1 and rec["tokens_per_s"] == 5.0


class _DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode()

    def get(self, k):
        return self.d[k]


def test_watchdog_and_heartbeat_report_instead_of_hanging():
    wd = StepWatchdog(0.05)
    assert wd.wait_until(lambda: True) < 0.05
    with pytest.raises(CommTimeout):
        wd.wait_until(lambda: False, what="never")
    store = _DictStore()
    a, b = Heartbeat(store, 0, 2), Heartbeat(store, 1, 2)
    a.beat(); b.beat()
    assert a.stale_ranks(0.02) == []
    time.sleep(0.03)
    b.beat()
    assert a.stale_ranks(0.02) == []                          # rank 1 moved
    time.sleep(0.03)
    assert a.stale_ranks(0.02) == [1]                         # rank 1 stopped: seen on the host, before any launch
    with pytest.raises(CommTimeout):
        a.check(0.02)


def test_cli_reproduces_the_documented_oracle_losses(capsys):
    from nano_megatron_b200.cli.run_reference_gpt import main
    assert main(["--gelu", "--learned-pos", "--tied", "--steps", "3", "--capture", "minimal"]) == 0
    out = capsys.readouterr().out
    losses = [float(line.split()[-1]) for line in out.strip().splitlines()]
    want = [42.140682, 40.074123, 37.985565]                  # the reference's own CPU run of this config
    assert all(abs(a - b) < 2e-4 for a, b in zip(losses, want)), losses


if __name__ == "__main__":
    from tests._dist_utils import run_worker_if_requested
    run_worker_if_requested(globals())


def test_nvtx_ranges_are_inert_without_cuda_and_toggle():
    from nano_megatron_b200.utils import tracing

    was = tracing.enabled()
    try:
        tracing.enable(True)
        assert tracing.enabled()
        with tracing.nvtx_range("phase"):   # no CUDA here: must not raise
            pass
        tracing.enable(False)
        assert not tracing.enabled()
        with tracing.nvtx_range("phase"):
            pass
    finally:
        tracing.enable(was)
