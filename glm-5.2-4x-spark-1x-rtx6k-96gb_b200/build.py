"""Build libglmrt_b200.so in-tree with nvcc for sm_100a.

    python build.py            # incremental: only stale objects are recompiled
    python build.py --force
    python build.py --trace    # libglmrt_b200_trace.so: the same library with the prefill GEMM's
                               # in-kernel timeline stamps compiled in (see trace_prefill.py)

The shared library lands beside this file; object files go to ``build/``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libglmrt_b200.so")
TRACE_LIB = os.path.join(HERE, "libglmrt_b200_trace.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libglmrt_b200.so cannot be built")
    return exe


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime() -> float:
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hdrs.append(os.path.join(HERE, "..", "include", "glmrt_b200.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    obj_dir = OBJ + "_trace" if trace else OBJ
    lib = TRACE_LIB if trace else LIB
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    hdr_time = _deps_mtime()
    jobs = []
    objs = []
    for src in _sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(obj_dir, src[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time):
            extra = ["-Xptxas", "-v"] if verbose else []
            if trace:
                extra.append("-DGLMRT_B200_TRACE")
            jobs.append([nvcc, *NVCC_FLAGS, *extra, "-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(run, jobs):
                if verbose and out:
                    print(out)
    if jobs or not os.path.exists(lib):
        run([nvcc, "-shared", "-o", lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
             "-Xcompiler", "-fPIC", "-cudart", "static", "-ldl"])
    return lib


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv)
    print(path)
