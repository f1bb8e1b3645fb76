"""Builds libf2k_attn.so (the CUDA kernels, the C ABI and the C++ call surface) in-tree.

The library holds sm_100a code only. It is compiled with nvcc directly, so it can be
cross-compiled on a machine without a GPU; `python -m f2k_cuda_b200.build` rebuilds it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "_build"
LIB_PATH = BUILD_DIR / "libf2k_attn.so"

SOURCES = ["attn_fwd_sm100.cu", "qk_prologue.cu", "capi.cu", "no_alloc.cu", "seqpar.cu", "headswap.cu", "f2k_compat.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the sm_100a library cannot be built")
    return cand


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) \
        + list(CSRC.rglob("*.cpp")) + [REPO_DIR / "include" / "f2k_attn.h", Path(__file__)]
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources; return its path.
    Safe to call from several processes at once (the ranks of a multi-GPU job all import the
    package): one builds under a file lock, the others wait and find the library fresh."""
    if not force and not _stale():
        return LIB_PATH
    BUILD_DIR.mkdir(exist_ok=True)
    import fcntl
    with open(BUILD_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _stale():       # another process built it while this one waited
                return LIB_PATH
            return _build_locked(verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(verbose: bool) -> Path:
    nvcc = _nvcc()
    objs = []
    for src in SOURCES:
        obj = BUILD_DIR / (src.rsplit(".", 1)[0] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-I", str(REPO_DIR / "include"), "-I", str(CSRC),
               "-I", str(CSRC / "compat"), "-DF2K_ATTN_BUILD", "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), file=sys.stderr)
        subprocess.run(cmd, check=True)
        objs.append(str(obj))
    tmp = LIB_PATH.with_suffix(".so.tmp")       # linked beside the target, then moved into place in one step
    cmd = [nvcc, "-shared", "-o", str(tmp), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(cmd, check=True)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
