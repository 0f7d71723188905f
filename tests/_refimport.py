"""Locate the unmodified reference package (for oracle-parity tests).

It is looked for in ``baseline/_ref`` (an offline ``pip install --target`` of
the reference) and, failing that, in ``/root/reference``.  Tests that need it
are skipped when it is absent.
"""
from __future__ import annotations

import importlib
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def reference_package():
    for cand in (os.path.join(ROOT, "baseline", "_ref"), "/root/reference"):
        if os.path.isdir(os.path.join(cand, "nano_megatron")):
            if cand not in sys.path:
                sys.path.append(cand)
            try:
                return importlib.import_module("nano_megatron")
            except Exception:  # pragma: no cover
                continue
    return None
