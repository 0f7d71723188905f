"""Ahead-of-time build of the sm_100a kernel library.

Every ``csrc/*.cu`` file is compiled with ``nvcc -gencode
arch=compute_100a,code=sm_100a`` into an object file and the objects are linked
into one shared library, ``nano_megatron_b200/libnmb_kernels.so``, which
:mod:`nano_megatron_b200.ops.native` loads with :mod:`ctypes`.  The library
sits in the source tree (it is git-ignored) so that a snapshot of the tree
carries it to a machine that has a GPU but has not built anything.

The reference project has no native code and therefore no build step
(``pyproject.toml`` there lists no extension modules); this file has no
counterpart in it.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC_DIR = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "csrc" / "build"
LIB_PATH = PKG_DIR / "libnmb_kernels.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the sm_100a kernels cannot be built")
    return exe


def _digest(path: Path) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    for header in sorted(SRC_DIR.glob("*.cuh")) + sorted(SRC_DIR.glob("*.h")):
        h.update(header.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(src: Path, force: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    digest = _digest(src)
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    stamp.write_text(digest)
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link the kernel library; returns its path."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(SRC_DIR.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no .cu sources under {SRC_DIR}")
    logs: list[str] = []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        results = list(pool.map(lambda s: _compile_one(s, force), sources))
    objs = [str(o) for o, _ in results]
    rebuilt = any(log for _, log in results)
    for src, (_, log) in zip(sources, results):
        if log:
            logs.append(f"==== {src.name}\n{log}")
    if rebuilt or force or not LIB_PATH.exists():
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *objs, "-lcudart"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    if logs:
        (OBJ_DIR / "ptxas.log").write_text("\n".join(logs))
        if verbose:
            print("\n".join(logs))
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
