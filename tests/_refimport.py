"""Locate the unmodified reference package (for oracle-parity tests).

It is looked for in ``baseline/_ref`` (an offline ``pip install --target`` of
the reference) and, failing that, in the directory named by the environment
variable ``NANO_MEGATRON_REFERENCE`` (a checkout of the reference).  Tests that
need it are skipped when it is absent.
"""
from __future__ import annotations

import importlib
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_package():
    cands = [os.path.join(ROOT, "baseline", "_ref")]
    if os.environ.get("NANO_MEGATRON_REFERENCE"):
        cands.append(os.environ["NANO_MEGATRON_REFERENCE"])
    for cand in cands:
        if os.path.isdir(os.path.join(cand, "nano_megatron")):
            if cand not in sys.path:
                sys.path.append(cand)
            try:
                return importlib.import_module("nano_megatron")
            except Exception:  # pragma: no cover
                continue
    return None
