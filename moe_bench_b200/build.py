"""Build ``libmoe_bench_b200.so`` in-tree with nvcc for sm_100a.

    python -m moe_bench_b200.build [--force] [--verbose]

The library is rebuilt when a source under ``csrc/`` or the public header is
newer than the existing ``.so``.  No GPU is needed to build.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ_DIR = os.path.join(PKG, "build")
LIB_PATH = os.path.join(PKG, "libmoe_bench_b200.so")
SOURCES = ["api.cu", "route_align.cu", "rows.cu", "grouped_gemm.cu", "grouped_gemm_fp8.cu", "grouped_gemm_fp8_cols.cu", "peer.cu", "dist.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "--extended-lambda",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def _inputs() -> list:
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(ROOT, "include", "moe_bench_b200.h"))
    return files


def needs_build() -> bool:
    return not _up_to_date(LIB_PATH)


def _up_to_date(path: str) -> bool:
    if not os.path.exists(path):
        return False
    built = os.path.getmtime(path)
    return not any(os.path.getmtime(f) > built for f in _inputs())


def build(force: bool = False, verbose: bool = False, variant: str = "", defines=()) -> str:
    """Build the library.  ``variant`` / ``defines`` build a differently named copy with
    extra ``-D`` flags (``libmoe_bench_b200_<variant>.so``), for comparing two builds side by side."""
    lib_path = LIB_PATH if not variant else os.path.join(PKG, f"libmoe_bench_b200_{variant}.so")
    obj_dir = OBJ_DIR if not variant else os.path.join(PKG, "build", variant)
    if not force and _up_to_date(lib_path):
        return lib_path
    nvcc = _nvcc()
    os.makedirs(obj_dir, exist_ok=True)
    extra = (["-Xptxas", "-v"] if verbose else []) + [f"-D{d}" for d in defines]

    def compile_one(src: str) -> str:
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    link = [nvcc, "-shared", "-o", lib_path, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    return lib_path


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
