"""Compiles oracle_c.c (the plain-C checker) into oracle/_build/liboracle_c.so and loads it with ctypes.
Test infrastructure only."""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_float, c_int, c_int64, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "oracle_c.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "liboracle_c.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    subprocess.run(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC", "-o", LIB, SRC, "-lm"],
                   check=True)
    return LIB


def load():
    lib = ctypes.CDLL(build())
    P = c_void_p
    lib.oc_absmax_scale.argtypes, lib.oc_absmax_scale.restype = [P, c_int64], c_float
    lib.oc_quantize.argtypes = [P, c_int64, c_float, c_int, c_uint64, c_uint64, P]
    lib.oc_igemm_nt.argtypes = [P, P, c_int64, c_int64, c_int64, P]
    lib.oc_spmm_copy_u.argtypes = [P, P, c_int64, P, c_int64, c_float, P]
    lib.oc_spmm_u_mul_e.argtypes = [P, P, P, c_int64, P, c_int64, c_int64, P, c_float, P]
    lib.oc_sddmm_dot.argtypes = [P, P, c_int64, P, P, c_int64, c_int64, c_float, c_float, P]
    return lib


if __name__ == "__main__":
    print(build(force=True))
