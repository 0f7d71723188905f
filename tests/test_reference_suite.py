"""The reference's OWN test-suite, unmodified, run against this package.

A checkout of the reference (with its ``tests/`` directory) is needed: point the
environment variable ``NANO_MEGATRON_REFERENCE`` at it; without it these tests are skipped.
The suite is copied to a temporary directory and started in a subprocess in which the
import name ``nano_megatron`` (and every submodule, ``nano_megatron.model`` included)
resolves to ``nano_megatron_b200``; child processes started by the suite (torchrun, Gloo)
inherit the alias through ``sitecustomize``.

What is allowed to fail, and why, is listed in ``EXPECTED_UNIT_FAILURES``.
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

ALIAS = '''
import importlib, importlib.abc, importlib.util, os, sys
_HERE = os.path.dirname(os.path.abspath(__file__))
if {root!r} not in sys.path:
    sys.path.append({root!r})
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)


class _Alias(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path=None, target=None):
        if name == "nano_megatron" or name.startswith("nano_megatron."):
            return importlib.util.spec_from_loader(name, self)
        return None

    def create_module(self, spec):
        return importlib.import_module("nano_megatron_b200" + spec.name[len("nano_megatron"):])

    def exec_module(self, module):
        pass


if not any(type(f).__name__ == "_Alias" for f in sys.meta_path):
    sys.meta_path.insert(0, _Alias())
'''

#: reference unit tests that do not pass against this package, with the reason
EXPECTED_UNIT_FAILURES = {
    # wording of an error message: flash attention here is bf16 only, the reference's text says "float16 or bfloat16"
    "test_resolve_flash_hard_fail_fp32",
    # counts a size-1 all-reduce that RowParallelLinear skips here when tp_size == 1 (a documented difference)
    "test_row_parallel_forward_one_all_reduce",
    # bit-for-bit comparison with a fixture recorded on another machine; the reference itself fails it here
    "test_golden_trajectory_fixture_strict",
    # MagicMock backends have every attribute, so the non-blocking ``isend`` path is taken instead of ``send``
    "test_send_forward_calls_backend", "test_send_backward_calls_backend",
}


def _checkout():
    path = os.environ.get("NANO_MEGATRON_REFERENCE")
    if not path or not os.path.isdir(os.path.join(path, "tests", "unit")):
        pytest.skip("NANO_MEGATRON_REFERENCE does not point at a checkout of the reference with its tests")
    return path


def _stage(checkout: str, tmp_path) -> str:
    work = str(tmp_path / "ref")
    shutil.copytree(os.path.join(checkout, "tests"), os.path.join(work, "tests"))
    open(os.path.join(work, "tests", "__init__.py"), "a").close()   # a regular package: not shadowed by this repo's tests/
    for name in ("conftest.py", "sitecustomize.py"):
        with open(os.path.join(work, name), "w") as f:
            f.write(ALIAS.format(root=ROOT))
    return work


def _run(work: str, targets: list[str], timeout: int):
    env = dict(os.environ, PYTHONPATH=work, MASTER_ADDR="127.0.0.1")
    proc = subprocess.run([sys.executable, "-m", "pytest", *targets, "-q", "-p", "no:cacheprovider", "--no-header",
                           "-W", "ignore"], cwd=work, env=env, capture_output=True, text=True, timeout=timeout)
    out = proc.stdout + proc.stderr
    failed = set(re.findall(r"^(?:FAILED|ERROR) \S+?::(?:\S+::)?(\w+)", out, flags=re.M))
    collect_errors = re.findall(r"^ERROR (\S+\.py)\s*$", out, flags=re.M)
    passed = re.search(r"(\d+) passed", out)
    return failed, collect_errors, int(passed.group(1)) if passed else 0, out


def test_reference_unit_tests_pass_against_this_package(tmp_path):
    work = _stage(_checkout(), tmp_path)
    failed, collect_errors, passed, out = _run(work, ["tests/unit"], 1200)
    assert not collect_errors, out[-3000:]
    assert failed <= EXPECTED_UNIT_FAILURES, (sorted(failed - EXPECTED_UNIT_FAILURES), out[-3000:])
    assert passed >= 170, out[-2000:]


def test_reference_gloo_and_integration_tests_pass_against_this_package(tmp_path):
    work = _stage(_checkout(), tmp_path)
    failed, collect_errors, passed, out = _run(work, ["tests/distributed", "tests/integration"], 2400)
    assert not collect_errors and not failed, out[-3000:]
    assert passed >= 10, out[-2000:]
