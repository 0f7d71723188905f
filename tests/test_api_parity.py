"""Every public name of the reference's five packages exists here, with every public method
of every exported class and every parameter of every signature (extra parameters with
defaults are allowed).  Skipped when the reference package is not installed."""
from __future__ import annotations

import importlib
import inspect

import pytest

from tests._refimport import reference_package

PAIRS = [("parallel", "parallel"), ("distributed", "distributed"), ("model", "models"), ("model", "model"),
         ("schedules", "schedules"), ("reference", "reference")]


def _params(obj):
    try:
        return list(inspect.signature(obj).parameters.values())
    except (TypeError, ValueError):
        return None


@pytest.mark.parametrize("ref_pkg,own_pkg", PAIRS, ids=[f"{a}->{b}" for a, b in PAIRS])
def test_public_api_of_the_reference_is_present(ref_pkg, own_pkg):
    if reference_package() is None:
        pytest.skip("reference package not installed")
    ref = importlib.import_module(f"nano_megatron.{ref_pkg}")
    own = importlib.import_module(f"nano_megatron_b200.{own_pkg}")
    problems = []
    for name in ref.__all__:
        theirs, ours = getattr(ref, name), getattr(own, name, None)
        if ours is None:
            problems.append(f"missing {name}")
            continue
        todo = [(name, theirs, ours)]
        if inspect.isclass(theirs):
            for meth, fn in inspect.getmembers(theirs, predicate=inspect.isfunction):
                if meth.startswith("_") and meth != "__init__":
                    continue
                mine = getattr(ours, meth, None)
                if mine is None:
                    problems.append(f"missing {name}.{meth}")
                else:
                    todo.append((f"{name}.{meth}", fn, mine))
        for label, a, b in todo:
            pa, pb = _params(a), _params(b)
            if pa is None or pb is None:
                continue
            have = {p.name for p in pb}
            takes_kwargs = any(p.kind == p.VAR_KEYWORD for p in pb)
            for p in pa:
                if p.kind in (p.VAR_KEYWORD, p.VAR_POSITIONAL) or p.name in have or takes_kwargs:
                    continue
                problems.append(f"{label} lacks parameter {p.name!r}")
    assert not problems, problems
