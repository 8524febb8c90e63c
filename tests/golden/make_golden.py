"""Generates tests/golden/primitives.npz: small seeded inputs with the outputs of the CPU oracle.

The reference has no golden vectors and its CUDA-only kernels cannot run where this script runs, so these fixtures
pin the *oracle* (regression) and give the GPU tests a second, file-based expectation.  The only inputs that come
from the reference are the two recipes it keeps under #ifdef TEST, reproduced by formula in oracle/tango_oracle.py.
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import tango_oracle as O  # noqa: E402


def main():
    rng = np.random.default_rng(20240)
    out = {}
    x = (rng.standard_normal((37, 41)) * 2.5).astype(np.float32)
    out["q_x"] = x
    out["q_scale"] = np.array([O.absmax_scale(x)], dtype=np.float32)
    for mode, name in ((0, "trunc"), (1, "nearest"), (2, "stoch")):
        out[f"q_{name}"] = O.quantize(x, out["q_scale"][0], mode, seed=42, call=7)
    # GEMM on the reference's TEST recipe
    a, b, sa, sb = O.recipe_gemm_inputs(64, 48, 96)
    y, aq, bq, *_ = O.qgemm_forward(a, b, sx=sa, sw=sb)
    out["gemm_a"], out["gemm_b"], out["gemm_y"], out["gemm_aq"], out["gemm_bq"] = a, b, y, aq, bq
    dyq = rng.integers(-127, 128, (64, 48), dtype=np.int8)
    out["gemm_dyq"] = dyq
    out["gemm_dx"] = O.qgemm_backward_dx(dyq, bq, np.float32(0.25), sb)
    out["gemm_dw"] = O.qgemm_backward_dw(dyq, aq, np.float32(0.25), sa)
    # small graph
    n, e = 40, 300
    src = rng.integers(0, n, e).astype(np.int64)
    dst = rng.integers(0, n, e).astype(np.int64)
    order = np.lexsort((src, dst))
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(indptr, dst + 1, 1)
    indptr = np.cumsum(indptr)
    out["g_src"], out["g_dst"], out["g_indptr"], out["g_indices"], out["g_eids"] = src, dst, indptr, src[order], order
    nq = rng.integers(-127, 128, (n, 4, 16), dtype=np.int8)
    eq = rng.integers(-127, 128, (e, 4), dtype=np.int8)
    out["g_nq"], out["g_eq"] = nq, eq
    out["spmm_copy_u"] = O.spmm_copy_u(indptr, src[order], nq, np.float32(0.02))
    out["spmm_u_mul_e"] = O.spmm_u_mul_e(indptr, src[order], order, nq, eq, np.float32(0.001))
    out["spmm_incidence"] = O.spmm_incidence(indptr, order, eq, np.float32(0.5))
    out["sddmm_dot"] = O.sddmm_dot(src, dst, nq, nq[::-1].copy(), np.float32(0.1), np.float32(0.2))
    out["sddmm_add"] = O.sddmm_elementwise("add", src, dst, eq[:n], eq[n:2 * n], np.float32(0.1), np.float32(0.2))
    # SDDMM recipe of the reference
    s2, d2, u2, v2, su, sv = O.recipe_sddmm_inputs(16)
    out["recipe_sddmm_add"] = O.sddmm_elementwise("add", s2, d2, u2, v2, su, sv)
    out["recipe_sddmm_dot"] = O.sddmm_dot(s2, d2, u2, v2, su, sv)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "primitives.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
