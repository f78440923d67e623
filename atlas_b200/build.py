"""Builds the native libraries in-tree with nvcc / g++ (no JIT cache):

* ``atlas_b200/_C/libatlas_b200_kernels.so``  — every ``csrc/*.cu`` compiled for sm_100a
* ``atlas_b200/_C/libatlas_b200_runtime.so``  — host runtime (``csrc/runtime/*.cpp``)
* ``atlas_b200/_C/libatlas_b200_bench.so``    — kernels that only the benchmarks use (``bench/csrc/*.cu``: memory-stream
  probes), kept out of the library the engine loads

``python -m atlas_b200.build`` rebuilds what is out of date.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "_C")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
KERNEL_LIB = os.path.join(OUT, "libatlas_b200_kernels.so")
RUNTIME_LIB = os.path.join(OUT, "libatlas_b200_runtime.so")
BENCH_CSRC = os.path.join(HERE, "bench", "csrc")
BENCH_LIB = os.path.join(OUT, "libatlas_b200_bench.so")


def _nvcc() -> str:
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _newer(src: str, dst: str, extra: List[str]) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(f) > t for f in [src] + extra)


def _run(cmd: List[str]) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout)


def build_kernels(verbose: bool = False, ptxas_v: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    cus = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    objs, jobs = [], []
    for f in cus:
        src = os.path.join(CSRC, f)
        obj = os.path.join(OUT, f[:-3] + ".o")
        objs.append(obj)
        if _newer(src, obj, headers):
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_v else []) + ["-I", CSRC, "-c", src, "-o", obj]
            jobs.append(cmd)
    if jobs:
        if verbose:
            print(f"[atlas_b200.build] compiling {len(jobs)} CUDA file(s) for sm_100a", file=sys.stderr)
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    if jobs or not os.path.exists(KERNEL_LIB):
        _run([_nvcc(), "-shared", "-o", KERNEL_LIB] + objs + ["-lcudart"])
    return KERNEL_LIB


def build_runtime(verbose: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    rdir = os.path.join(CSRC, "runtime")
    if not os.path.isdir(rdir):
        return ""
    srcs = sorted(os.path.join(rdir, f) for f in os.listdir(rdir) if f.endswith(".cpp"))
    hdrs = [os.path.join(rdir, f) for f in os.listdir(rdir) if f.endswith(".h")]
    if not srcs:
        return ""
    if any(_newer(s, RUNTIME_LIB, hdrs) for s in srcs):
        if verbose:
            print("[atlas_b200.build] compiling host runtime", file=sys.stderr)
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", RUNTIME_LIB] + srcs)
    return RUNTIME_LIB


def build_bench(verbose: bool = False) -> str:
    """Benchmark-only kernels; they use the kernel library's tensor-map helper, so that library is linked in."""
    if not os.path.isdir(BENCH_CSRC):
        return ""
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    cus = sorted(f for f in os.listdir(BENCH_CSRC) if f.endswith(".cu"))
    objs, stale = [], False
    for f in cus:
        src, obj = os.path.join(BENCH_CSRC, f), os.path.join(OUT, "bench_" + f[:-3] + ".o")
        objs.append(obj)
        if _newer(src, obj, headers):
            if verbose:
                print(f"[atlas_b200.build] compiling bench/csrc/{f}", file=sys.stderr)
            _run([_nvcc()] + NVCC_FLAGS + ["-I", CSRC, "-c", src, "-o", obj])
            stale = True
    if objs and (stale or not os.path.exists(BENCH_LIB)):
        _run([_nvcc(), "-shared", "-o", BENCH_LIB] + objs + ["-L", OUT, "-latlas_b200_kernels", "-Xlinker", "-rpath=$ORIGIN",
                                                             "-lcudart"])
    return BENCH_LIB


def build_all(verbose: bool = True) -> None:
    build_kernels(verbose)
    build_runtime(verbose)
    build_bench(verbose)


if __name__ == "__main__":
    build_all(True)
    print(KERNEL_LIB)
