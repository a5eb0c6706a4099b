"""Builds libxg_sm100.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

Usage: ``python -m xpu_graph_b200.build [--force] [--verbose]``.
Objects go to ``xpu_graph_b200/csrc/build/``; the shared library lands next to this file so that it
travels with the source tree. Nothing here needs a GPU: nvcc cross-compiles.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(HERE, "libxg_sm100.so")

SOURCES = [
    "abi.cu",
    "norm.cu",
    "elementwise.cu",
    "copy_fusions.cu",
    "gemm.cu",
    "gemm_tc.cu",
    "gemm_tc_ksplit.cu",
    "gemm_mlp.cu",
    "mlp_small.cu",
    "gemm_f32.cu",
    "split_bf16x3.cu",
    "sdpa.cu",
    "sum3d.cu",
    "rowsum_cat.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _deps_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths.append(os.path.join(HERE, "..", "include", "xg_sm100.h"))
    paths.append(os.path.abspath(__file__))
    return max(os.path.getmtime(p) for p in paths)


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr if verbose else ""


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every kernel source and link the shared library. Returns the library path."""
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_time = _deps_mtime()
    jobs = []
    objs = []
    for name in SOURCES:
        src = os.path.join(CSRC, name)
        obj = os.path.join(OBJ_DIR, name.replace(".cu", ".o"))
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, verbose) for s, o in jobs]
            for f in futs:
                out = f.result()
                if out:
                    print(out, file=sys.stderr)
    need_link = bool(jobs) or not os.path.exists(LIB_PATH)
    if need_link:
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
