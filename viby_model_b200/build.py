"""Build recipe for libvc1d.so: nvcc, sm_100a only, in-tree output next to this file.

Run as ``python viby_model_b200/build.py`` (add ``--force`` to rebuild everything,
``--verbose`` for ptxas register/spill reports).  Objects go to ``build/vc1d`` at the
repository root; the shared library is written to ``viby_model_b200/libvc1d.so``.
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
REPO = PKG_DIR.parent
OBJ_DIR = REPO / "build" / "vc1d"
LIB_PATH = PKG_DIR / "libvc1d.so"

SOURCES = [
    "api.cu",
    "prefill_channel_last.cu",
    "prefill_time_major.cu",
    "prefill_generic.cu",
    "prefill_tma.cu",
    "prefill_tma_f32.cu",
    "prefill_tma_bf16.cu",
    "prefill_tma_f16.cu",
    "prefill_noalloc.cu",
    "prefill_bwd_generic.cu",
    "prefill_bwd_tma.cu",
    "prefill_bwd_tma_f32.cu",
    "prefill_bwd_tma_bf16.cu",
    "prefill_bwd_tma_f16.cu",
    "update.cu",
    "update_bwd.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put the CUDA 12.9 toolkit on PATH")


def _deps_mtime() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [REPO / "include" / "vc1d.h", Path(__file__)]
    return max(h.stat().st_mtime for h in headers)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every translation unit (in parallel) and link libvc1d.so. Returns its path."""
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr_m = _deps_mtime()
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(name: str):
        src = CSRC / name
        obj = OBJ_DIR / (src.stem + ".o")
        if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_m):
            return obj, ""
        cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {name}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr

    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 4)) as ex:
        results = list(ex.map(compile_one, SOURCES))
    objs = [str(o) for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    newest = max(Path(o).stat().st_mtime for o in objs)
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest:
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcuda"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
