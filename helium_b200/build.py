"""Builds libhelium_b200.so (sm_100a only) in-tree with nvcc.

    python helium_b200/build.py [--force] [--verbose] [--ptxas]

(run by path: importing the package requires the library this script produces)

The library is the product: the Python package refuses to work without it.  Objects are rebuilt
only when their source (or any header) is newer than the object.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
INCLUDE = os.path.join(os.path.dirname(ROOT), "include")
OBJ_DIR = os.path.join(ROOT, "build")
LIB_DIR = os.path.join(ROOT, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libhelium_b200.so")

SOURCES = [
    "api.cu",
    "permute.cu",
    "pointwise_compile.cu",
    "pointwise.cu",
    "pointwise_dense.cu", "pointwise_jit.cu",
    "gemm_plan.cu",
    "gemm_kernels_flex.cu",
    "gemm_kernels_c3.cu",
    "gemm_kernels_prog.cu",
    "sgemm.cu",
    "host_graph.cu",
    "fusion_search.cu",
    "reduce_noalloc.cu",
    "comm.cu",
    "conv.cu",
    "train_ops.cu",
]

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-I", INCLUDE,
    "-I", CSRC,
    "-DHE_BUILDING_LIBRARY",
]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _newest_header_mtime() -> float:
    newest = 0.0
    for d in (CSRC, INCLUDE):
        for name in os.listdir(d):
            if name.endswith((".h", ".cuh")):
                newest = max(newest, os.path.getmtime(os.path.join(d, name)))
    return newest


def _compile(nvcc: str, src: str, obj: str, verbose: bool, ptxas_v: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
    if ptxas_v:
        cmd += ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return (res.stdout + res.stderr) if (verbose or ptxas_v) else ""


def build(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> str:
    nvcc = nvcc_path()
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    hdr_mtime = _newest_header_mtime()
    jobs = []
    objs = []
    for name in SOURCES:
        src = os.path.join(CSRC, name)
        if not os.path.exists(src):
            raise RuntimeError(f"missing source {src}")
        obj = os.path.join(OBJ_DIR, name.replace(".cu", ".o"))
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_mtime)
        if stale:
            jobs.append((src, obj))
    logs = []
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose, ptxas_v), jobs):
                if out:
                    logs.append(out)
    need_link = bool(jobs) or not os.path.exists(LIB_PATH)
    if need_link:
        cmd = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if logs:
        print("\n".join(logs))
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_v="--ptxas" in sys.argv)
    print(path)
