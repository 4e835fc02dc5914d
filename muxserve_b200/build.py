"""In-tree build of ``libmuxb200.so`` (CUDA kernels + host C++ behind the C ABI).

``python -m muxserve_b200.build`` compiles every source under ``csrc/`` for
sm_100a with nvcc and links one shared library next to this file.  nvcc
cross-compiles, so no GPU is needed to build.  The library is never built
implicitly at import time on a machine without nvcc: loading fails loudly.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libmuxb200.so"
BUILD_DIR = PKG_DIR / "build"

CUDA_SOURCES = ["status.cu", "cache_write.cu", "rotary.cu", "block_table.cu", "paged_attention.cu",
                "prefill_attention.cu", "tp_allreduce.cu", "oproj_allreduce.cu"]
HOST_SOURCES = ["host/kv_storage.cpp", "host/batch_scheduler.cpp"]
HEADERS = ["ptx.cuh", "internal.h", "attn_common.cuh", "rope.cuh", "../../include/muxb200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--use_fast_math",
]
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: cannot build libmuxb200.so")
    return cand


def all_sources():
    return [CSRC / s for s in CUDA_SOURCES + HOST_SOURCES + HEADERS]


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(src.stat().st_mtime > built for src in all_sources())


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    res = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(str(c) for c in cmd)}\n{res.stdout}\n{res.stderr}")
    if verbose and (res.stdout or res.stderr):
        print(res.stdout, res.stderr, sep="\n", flush=True)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile and link the library if it is missing or older than a source."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = _nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    jobs = []
    objs = []
    for src in CUDA_SOURCES:
        obj = BUILD_DIR / (Path(src).stem + ".o")
        flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
        jobs.append([nvcc, *flags, "-c", CSRC / src, "-o", obj])
        objs.append(obj)
    for src in HOST_SOURCES:
        obj = BUILD_DIR / (Path(src).stem + ".o")
        jobs.append(["g++", *HOST_FLAGS, "-c", CSRC / src, "-o", obj])
        objs.append(obj)
    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as pool:
        list(pool.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    _run([nvcc, "-shared", "-o", tmp, *objs, "-cudart", "static"], verbose)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
