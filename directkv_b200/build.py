"""In-tree build of libdirectkv_b200.so (sm_100a only) with nvcc.

Usage: ``python -m directkv_b200.build [-v]``.  The shared object lands next to the package
(``directkv_b200/_lib/``) so that it travels with the source tree; nothing is installed into
site-packages and nothing is JIT-compiled at import time.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "_lib"
LIB_PATH = LIB_DIR / "libdirectkv_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-shared",
    "-cudart", "static",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def sources():
    return [CSRC / "dkv_capi.cu", CSRC / "dkv_noalloc.cu"]


def headers():
    return sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "directkv_b200.h"]


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > t for p in list(sources()) + list(headers()))


def build_library(verbose: bool = False, force: bool = False) -> Path:
    """Compiles the CUDA sources when the library is missing or older than a source file."""
    if not force and not is_stale():
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [find_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB_PATH), *map(str, sources())]
    env = dict(os.environ)
    # nvcc needs a host compiler it supports; the distribution's g++ is the one it was tested with.
    if os.path.exists("/usr/bin/g++"):
        cmd += ["-ccbin", "/usr/bin/g++"]
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libdirectkv_b200.so:\n" + proc.stderr[-4000:])
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(verbose="-v" in sys.argv, force=True)
    print(path)
