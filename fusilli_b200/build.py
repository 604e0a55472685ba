"""Builds libfusilli_b200.so in-tree with nvcc for sm_100a (no other target)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libfusilli_b200.so")
OBJ = os.path.join(HERE, "_obj")

SOURCES = [
    "runtime.cu",
    "comm.cu",
    "plan.cpp",
    "kernels/pointwise.cu",
    "kernels/reduce.cu",
    "kernels/norm.cu",
    "kernels/batchnorm.cu",
    "kernels/contract_simt.cu",
    "kernels/sdpa_simt.cu",
    "kernels/gemm_tc.cu",
    "kernels/conv_tc.cu",
    "kernels/conv_wgrad_tc.cu",
    "kernels/conv_split_f32.cu",
    "kernels/sdpa_tc.cu",
    "kernels/selftest.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "-x", "cu",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libfusilli_b200.so cannot be built")
    return exe


def _stale(obj: str, deps) -> bool:
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers():
    out = [os.path.join(HERE, "..", "include", "fusilli_b200.h")]
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".h", ".cuh"))]
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdrs = _headers()
    jobs = []
    objs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, src.replace("/", "_") + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + hdrs):
            extra = os.environ.get("FUSILLI_B200_NVCC_EXTRA", "").split()  # e.g. -DNAME for an instrumented build
            cmd = [nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for " + cmd[-3])

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(run, jobs))
    if jobs or not os.path.exists(LIB):
        link = [nvcc(), "-shared", "-o", LIB] + objs + ["-cudart", "static", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of libfusilli_b200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
