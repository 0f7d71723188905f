"""The allocation-free column-sum entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory when they call into
it (a fixed, pre-partitioned memory budget; a host framework that owns all
device memory; a loop that must not touch the allocator).  For them the library
carries its own scratch in a fixed ``__device__`` array.  This test calls
``nmb_col_sum_noalloc`` directly with ctypes -- no wrapper -- twice in a row on
different data and compares each result with the regular entry point (whose
scratch comes from the caller), then checks that an oversize request is refused.

The file name sorts last so that a run that stops at the first failure has
already executed every other test.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, dy, out, accumulate=0):
    rows, cols = dy.shape
    lib.nmb_col_sum_noalloc.restype = ctypes.c_int
    lib.nmb_col_sum_noalloc_strerror.restype = ctypes.c_char_p
    return lib.nmb_col_sum_noalloc(
        ctypes.c_void_p(dy.data_ptr()), ctypes.c_int(dy.stride(0)), ctypes.c_void_p(out.data_ptr()),
        ctypes.c_int(rows), ctypes.c_int(cols), ctypes.c_int(accumulate),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_col_sum_matches_regular_entry_point_twice():
    from nano_megatron_b200.ops import kernels, native

    lib = native.lib()
    torch.manual_seed(0)
    # two calls in a row, different shapes: the second must not see the first one's leftovers
    for rows, cols in ((4096, 1024), (777, 130)):
        dy = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
        want = kernels.col_sum(dy)
        got = torch.full((cols,), 7.0, dtype=torch.bfloat16, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = _call(lib, dy, got)
        assert rc == 0, lib.nmb_col_sum_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        ref = dy.float().sum(0)
        tol = 2e-2 * max(1.0, ref.abs().max().item())
        assert (got.float() - want.float()).abs().max().item() <= tol
        assert (got.float() - ref).abs().max().item() <= tol
    # accumulate flag and strided rows
    wide = torch.randn(512, 256, device="cuda").to(torch.bfloat16)
    view = wide[:, :128]
    acc = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    assert _call(lib, view, acc, accumulate=1) == 0
    torch.cuda.synchronize()
    ref = view.float().sum(0) + 1.0
    assert (acc.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())


def test_no_alloc_col_sum_rejects_oversize_and_odd_shapes():
    from nano_megatron_b200.ops import native

    lib = native.lib()
    lib.nmb_col_sum_noalloc_strerror.restype = ctypes.c_char_p
    limit = lib.nmb_col_sum_noalloc_max_cols()
    assert limit == 8192
    big = torch.zeros(4, limit + 2, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(limit + 2, dtype=torch.bfloat16, device="cuda")
    rc = _call(lib, big, out)
    assert rc == 4 and b"8192" in lib.nmb_col_sum_noalloc_strerror(rc)
    odd = torch.zeros(4, 6, dtype=torch.bfloat16, device="cuda")[:, :5]
    assert _call(lib, odd, out) == 3
    torch.cuda.synchronize()


def test_no_alloc_col_sum_rejects_misaligned_view_and_zeroes_on_no_rows():
    """A bf16 view that starts at an odd element (even pitch, even width) would be
    read with misaligned 4-byte loads: it must be refused before any launch."""
    from nano_megatron_b200.ops import native

    lib = native.lib()
    wide = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
    view = wide[:, 1:129]
    assert view.data_ptr() % 4 == 2 and view.stride(0) % 2 == 0 and view.shape[1] % 2 == 0
    out = torch.full((128,), 3.0, dtype=torch.bfloat16, device="cuda")
    rc = _call(lib, view, out)
    assert rc == 3 and b"aligned" in lib.nmb_col_sum_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert torch.all(out == 3.0)            # nothing was launched
    # no rows: the sum over nothing is zero (kept when accumulating)
    empty = wide[:0, :128]
    assert _call(lib, empty, out, accumulate=1) == 0
    torch.cuda.synchronize()
    assert torch.all(out == 3.0)
    assert _call(lib, empty, out) == 0
    torch.cuda.synchronize()
    assert torch.all(out == 0.0)
