"""Command-line tools that need no GPU: the architecture verifier and the
benchmark report writer (counterparts of the reference's
``scripts/verify_architecture.py`` and the report half of ``scripts/benchmark_tp.py``)."""
from __future__ import annotations

import io
import json

import pytest

from nano_megatron_b200.cli import benchmark, verify_architecture as va
from nano_megatron_b200.reference import gpt_preset


@pytest.mark.parametrize("name,params_m", [("345m", 355.9), ("760m", 760.4), ("1.3b", 1315.8)])
def test_closed_form_parameter_count_matches_the_module(name, params_m):
    cfg = gpt_preset(name, attn_backend="unfused")
    assert va.count_parameters(cfg) == va.expected_parameter_count(cfg)
    assert va.count_parameters(cfg) / 1e6 == pytest.approx(params_m, abs=0.1)


@pytest.mark.parametrize("over", [
    {}, dict(use_bias=False, tie_word_embeddings=False, position_embedding_type="rope", gated_linear_unit=True,
             activation_func="swiglu", vocab_size=51200),
    dict(num_query_groups=4, use_fused_qkv=False, normalization="rmsnorm"),
])
def test_verifier_accepts_every_knob_set(over):
    cfg = gpt_preset("small", attn_backend="unfused", **over)
    out = io.StringIO()
    assert va.verify(cfg, None, out=out)
    text = out.getvalue()
    assert "architecture matches" in text and "num_attention_heads" in text
    assert va.count_parameters(cfg) == va.expected_parameter_count(cfg)


def test_verifier_cli_exit_code():
    assert va.main(["--preset", "small", "--no-forward"]) == 0


def _line(impl, value, nopt, mem):
    return {"impl": impl, "value": value, "ms_per_step": 4096e3 / value, "n_gpus": 2, "peak_mem_mb": mem,
            "config": {"model": "GPT-345m", "global_batch": 4, "seq_len": 2048, "parallelism": "dp2"},
            "step_without_optimizer": {"value": nopt, "ms_per_step": 4096e3 / nopt}, "e2e": {"value": value * 0.99},
            "modes": {"tp2+sp-345m": {"config": {"model": "GPT-345m", "global_batch": 2, "seq_len": 2048,
                                                  "parallelism": "tp2+sp"}, "value": value / 2,
                                      "ms_per_step": 1.0, "peak_mem_mb": mem / 2,
                                      "step_without_optimizer": {"value": nopt / 2, "ms_per_step": 0.9}},
                      "broken": {"error": "boom"}}}


def test_report_writer_tables_and_ratios(tmp_path):
    lines = tmp_path / "runs.jsonl"
    lines.write_text(json.dumps(_line("b200", 400000.0, 450000.0, 9000.0)) + "\n"
                     + json.dumps(_line("reference", 100000.0, 150000.0, 12000.0)) + "\n"
                     + json.dumps({"impl": "reference", "unavailable": "x"}) + "\n")
    report = tmp_path / "performance.md"
    assert benchmark.main(["--from-json", str(lines), "--report", str(report)]) == 0
    text = report.read_text()
    assert text.count("| nano_megatron_b200 |") == 2 and text.count("| reference |") == 2
    assert "Peak memory (MB)" in text and "no optimizer" in text
    assert "dp2 on 2 GPU(s), GPT-345m: 4.00x with AdamW, 3.00x without; peak memory 0.75x" in text
    results = benchmark.results_from_json(_line("b200", 1.0, 2.0, 3.0))
    assert [r.parallelism for r in results] == ["dp2", "tp2+sp"]
