"""Helpers for multi-process tests: N local processes stand in for N nodes.

A launcher test spawns ``python -m torch.distributed.run`` on this file's
caller with an environment variable naming the worker function; rendezvous is on
127.0.0.1 with a port derived from the test id.  Gloo on CPU needs no GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER_ENV = "NMB_DIST_WORKER"


def port_for(test_id: str) -> int:
    return 29500 + int(hashlib.sha1(test_id.encode()).hexdigest(), 16) % 2000


def launch(script: str, worker: str, world: int, *, timeout: int = 300, extra_env: dict | None = None) -> str:
    """Run ``script`` under torchrun with ``world`` ranks; ``worker`` names the function to run."""
    env = dict(os.environ)
    env[WORKER_ENV] = worker
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    env.setdefault("OMP_NUM_THREADS", "1")
    if extra_env:
        env.update(extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr=127.0.0.1", f"--master-port={port_for(script + worker + str(world))}", script]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    for line in proc.stdout.splitlines():
        if line.startswith("PERF"):
            print(line)
    if proc.returncode != 0:
        tail = (proc.stdout[-3000:] + "\n" + proc.stderr[-6000:])
        raise AssertionError(f"distributed worker {worker} (world {world}) failed:\n{tail}")
    return proc.stdout


def run_worker_if_requested(namespace: dict) -> None:
    """Call at the bottom of a test module: under torchrun, run the named worker and exit."""
    name = os.environ.get(WORKER_ENV)
    if name and "RANK" in os.environ:
        namespace[name]()
        sys.exit(0)
