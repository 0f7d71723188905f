"""ctypes loader for the sm_100a kernel library.

The library is built by :mod:`nano_megatron_b200.build` and lives next to the
package as ``libnmb_kernels.so``.  On a machine with a CUDA device a missing
library is an error (the ops never fall back silently to PyTorch on a GPU);
without a device the library is simply not needed.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "libnmb_kernels.so"
_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()

STATUS_NAMES = {0: "ok", 1: "mbarrier wait timed out", 2: "peer flag wait timed out",
                3: "bad argument", 4: "size beyond the supported maximum"}


class NativeKernelError(RuntimeError):
    """A kernel launcher or a device-side bounded wait reported a failure."""


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


_configured_devices: set[int] = set()
_SPLITK_WS_BYTES = 64 << 20
_splitk_keep: dict[int, tuple] = {}


def _configure_current_device(loaded: ctypes.CDLL) -> None:
    """Shared-memory opt-ins of the big kernels are per device: set them the
    first time the library is used with a given device current."""
    if not torch.cuda.is_available():
        return
    dev = torch.cuda.current_device()
    if dev in _configured_devices:
        return
    for fn in (loaded.nmb_gemm_configure, loaded.nmb_attn_configure, loaded.nmb_norm_configure,
               loaded.nmb_comm_configure):
        rc = fn()
        if rc != 0:
            raise NativeKernelError(f"kernel configuration failed with code {rc} on device {dev}")
    if os.environ.get("NMB_SPLITK", "0") == "1":
        # Scratch of the split-K weight-gradient GEMMs (fp32 partial tiles + per-tile counters),
        # registered once per device so that the launchers never allocate.  Off by default: the
        # GPT-345M step (B2 x S2048, one GPU) measured 17.95 ms with it against 17.66 ms without;
        # the exchange of partial tiles costs more than the idle SMs of the 32- and 96-tile
        # weight gradients do.
        ws = torch.empty(_SPLITK_WS_BYTES // 4, dtype=torch.float32, device=torch.device("cuda", dev))
        counters = torch.zeros(1024, dtype=torch.int32, device=torch.device("cuda", dev))
        rc = loaded.nmb_gemm_set_splitk_workspace(ctypes.c_void_p(ws.data_ptr()), ctypes.c_longlong(_SPLITK_WS_BYTES),
                                                  ctypes.c_void_p(counters.data_ptr()), ctypes.c_int(counters.numel()))
        if rc != 0:
            raise NativeKernelError(f"split-K workspace registration failed with code {rc} on device {dev}")
        _splitk_keep[dev] = (ws, counters)
    _configured_devices.add(dev)


def enable_split_k(device_index: int, enabled: bool = True) -> None:
    """Register (or withdraw) the split-K workspace of ``device_index`` (which must be current)."""
    loaded = lib()
    if enabled:
        dev = torch.device("cuda", device_index)
        ws = torch.empty(_SPLITK_WS_BYTES // 4, dtype=torch.float32, device=dev)
        counters = torch.zeros(1024, dtype=torch.int32, device=dev)
        rc = loaded.nmb_gemm_set_splitk_workspace(ctypes.c_void_p(ws.data_ptr()), ctypes.c_longlong(_SPLITK_WS_BYTES),
                                                  ctypes.c_void_p(counters.data_ptr()), ctypes.c_int(counters.numel()))
        _splitk_keep[device_index] = (ws, counters)
    else:
        rc = loaded.nmb_gemm_set_splitk_workspace(None, ctypes.c_longlong(0), None, ctypes.c_int(0))
        _splitk_keep.pop(device_index, None)
    if rc != 0:
        raise NativeKernelError(f"split-K workspace registration failed with code {rc}")


def lib() -> ctypes.CDLL:
    """Load (once) and return the kernel library."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not _LIB_PATH.exists():
                    raise NativeKernelError(
                        f"{_LIB_PATH} is missing: run `python -m nano_megatron_b200.build` "
                        "(the CUDA ops do not fall back to PyTorch on a GPU)"
                    )
                _lib = ctypes.CDLL(str(_LIB_PATH))
                pair = os.environ.get("NMB_GEMM_PAIR")
                if pair is not None:
                    _lib.nmb_gemm_set_pair(int(pair != "0"))
                pdl = os.environ.get("NMB_PDL")      # "0": plain stream order for every kernel
                if pdl is not None:
                    _lib.nmb_set_pdl(int(pdl != "0"))
    _configure_current_device(_lib)
    return _lib


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr(device: torch.device | None = None) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels write on a timed-out wait."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def check_status(device: torch.device | None = None, *, reset: bool = True) -> None:
    """Read the status word (host sync) and raise if a kernel reported a failure."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    w = status_word(device)
    v = int(w.item())
    if v != 0:
        if reset:
            w.zero_()
        code, where = v & 0xFF, v >> 8
        raise NativeKernelError(
            f"device-side failure: {STATUS_NAMES.get(code, code)} (site {where})"
        )


#: kernels launched by each C entry point (for launch accounting)
_KERNELS_PER_CALL = {"nmb_attn_bwd": 3, "nmb_col_reduce": 2, "nmb_adamw_step": 2}
#: running count of kernels of this library launched (or captured) by this process
launches = 0
#: the same per C entry point (tests use it to show that a fused path left no stand-alone kernel behind)
launch_counts: dict[str, int] = {}


def check_rc(rc: int, what: str) -> None:
    global launches
    if rc != 0:
        raise NativeKernelError(f"{what}: launcher returned {rc}")
    launches += _KERNELS_PER_CALL.get(what, 1)
    launch_counts[what] = launch_counts.get(what, 0) + 1
