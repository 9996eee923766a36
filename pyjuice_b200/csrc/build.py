"""Builds the CUDA library in-tree: ``python -m pyjuice_b200.csrc.build``.

One shared object, ``libpcx_b200.so``, from every ``.cu`` file beside this script, compiled for
sm_100a only.  ``nvcc`` cross-compiles, so no GPU is needed to build.

``python -m pyjuice_b200.csrc.build --trace`` builds a second library, ``libpcx_b200_trace.so``, with
``-DPCX_TRACE``: the dataflow launch and the first-generation dense GEMM then stamp ``%globaltimer`` at the phases
of every tile into a device array that ``pcx_trace_read(host_buffer, n_items)`` copies out (12 int64 per tile).
Load it instead of the regular library with ``PCX_B200_LIB=<path>``; it is a development aid (the per-level and
per-chunk timings quoted in the design notes come from it) and is never loaded by default.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libpcx_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
         "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "*.cu")))


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(HERE, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "..", "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    if trace:
        return _build(os.path.join(HERE, "libpcx_b200_trace.so"), ["-DPCX_TRACE"], ".trace.o", verbose)
    if not force and not needs_build():
        return LIB
    return _build(LIB, [], ".o", verbose)


def _build(lib: str, extra, obj_suffix: str, verbose: bool) -> str:
    flags = [f for f in FLAGS if not f.startswith("--use_fast_math")] + list(extra)
    from concurrent.futures import ThreadPoolExecutor

    def compile_one(src):
        obj = src[:-3] + obj_suffix
        cmd = [NVCC, *flags, "-c", src, "-o", obj] + (["-Xptxas", "-v"] if verbose else [])
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=4) as pool:       # one nvcc per translation unit, side by side
        objs = list(pool.map(compile_one, sources()))
    subprocess.run([NVCC, "-shared", "-o", lib, *objs, "-lcudart"], check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
