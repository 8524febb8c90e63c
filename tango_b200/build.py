"""Builds the sm_100a shared library in-tree (tango_b200/lib/libtango_b200.so) with nvcc.

nvcc cross-compiles without a GPU.  The explicit -gencode pair is required: tcgen05 kind::i8 only assembles for the
architecture-specific target compute_100a/sm_100a.  --fmad=false keeps every fp32 epilogue a sequence of single
IEEE operations so results are bit-reproducible against the CPU checker.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libtango_b200.so")
SOURCES = ["quantize.cu", "spmm.cu", "sddmm.cu", "gat_softmax.cu", "igemm_tcgen05.cu", "peer.cu"]
# measurement aid of the benchmark, a library of its own (not part of the product ABI)
PROBE_SRC = os.path.join(CSRC, "bench", "row_gather_probe.cu")
PROBE_LIB_PATH = os.path.join(LIB_DIR, "libtango_bench_probe.so")


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(PROBE_LIB_PATH):
        return True
    t = min(os.path.getmtime(LIB_PATH), os.path.getmtime(PROBE_LIB_PATH))
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))]
    deps += [PROBE_SRC, os.path.join(ROOT, "include", "tango_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc(), "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
           "-O3", "--fmad=false", "-std=c++17", "-diag-suppress", "128", "-I", os.path.join(ROOT, "include"),
           "-o", LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libtango_b200.so")
    if verbose:
        sys.stderr.write(res.stderr)
    res = subprocess.run([_nvcc(), "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a",
                          "-lineinfo", "-O3", "-std=c++17", "-o", PROBE_LIB_PATH, PROBE_SRC],
                         capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libtango_bench_probe.so")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
