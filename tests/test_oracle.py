"""CPU tests of the oracle itself: published known answers, the reference's TEST recipes, independent
re-derivations (SciPy sparse products, the plain-C checker) and the committed golden file."""
import os

import numpy as np
import pytest
import scipy.sparse as sp
from hypothesis import given, settings, strategies as st

from oracle import c_oracle as C
from oracle import tango_oracle as O

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "primitives.npz"))


def test_philox_known_answers():
    """Known-answer vectors published with the Random123 library for philox4x32-10."""
    r = O.philox4x32_10(np.array([0], np.uint32), 0, 0, 0, 0, 0)
    assert [int(v[0]) for v in r] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    f = 0xFFFFFFFF
    r = O.philox4x32_10(np.array([f], np.uint32), f, f, f, f, f)
    assert [int(v[0]) for v in r] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    r = O.philox4x32_10(np.array([0x243F6A88], np.uint32), 0x85A308D3, 0x13198A2E, 0x03707344, 0xA4093822, 0x299F31D0)
    assert [int(v[0]) for v in r] == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_gemm_recipe_is_exact_integer_product():
    """With the reference's TEST inputs (integers in [-8,7], scales 0.5; cuda/src/QGEMM_forward.cu:162-210) the
    quantized product must equal the plain product A.B^T exactly -- the check that main() performs with cuBLAS."""
    a, b, sa, sb = O.recipe_gemm_inputs(96, 40, 64)
    y, aq, bq, *_ = O.qgemm_forward(a, b, sx=sa, sw=sb)
    np.testing.assert_array_equal(aq, (2 * a).astype(np.int8))
    np.testing.assert_array_equal(y, a @ b.T)


def test_sddmm_recipe_values():
    """cuda/src/SDDMM.cu:230-257: U[i] = i, V[i] = 3*dim - i, edges (0,0),(0,1),(0,2),(1,2), scales 1."""
    dim = 16
    src, dst, u, v, su, sv = O.recipe_sddmm_inputs(dim)
    add = O.sddmm_elementwise("add", src, dst, u, v, su, sv)
    for e, (s, d) in enumerate(zip(src, dst)):
        for j in range(dim):
            assert add[e, j] == (s * dim + j) + (3 * dim - (d * dim + j))
    dot = O.sddmm_dot(src, dst, u, v, su, sv)
    assert dot[0, 0] == sum(j * (48 - j) for j in range(16))


@settings(max_examples=60, deadline=None)
@given(st.lists(st.floats(-1e3, 1e3, width=32), min_size=1, max_size=64), st.integers(0, 2))
def test_quantizer_invariants(vals, mode):
    x = np.array(vals, dtype=np.float32)
    s = O.absmax_scale(x)
    q = O.quantize(x, s, mode, seed=3, call=1).astype(np.int32)
    assert np.all(np.abs(q) <= 127)
    if s == 0:
        assert np.all(q == 0)
        return
    t = (x * O.inv_scale(s)).astype(np.float32)
    if mode == O.ROUND_NEAREST:
        assert np.all(np.abs(q - t) <= 0.5 + 1e-6)
    elif mode == O.ROUND_TRUNC:
        assert np.all(np.abs(q) <= np.abs(t) + 1e-6) and np.all(np.abs(q - t) < 1 + 1e-6)
    else:
        lo, hi = np.clip(np.floor(t), -127, 127), np.clip(np.floor(t) + 1, -127, 127)
        assert np.all((q == lo) | (q == hi))
    np.testing.assert_array_equal(q.astype(np.int8), C.quantize(x, s, mode, 3, 1))


def test_stochastic_rounding_mean():
    x = np.full(200000, 0.3, dtype=np.float32)
    x[0] = 1.0
    q = O.quantize(x, O.absmax_scale(x), O.ROUND_STOCHASTIC, seed=1, call=2)
    assert abs(q[1:].mean() - 38.1) < 0.01


def _rand_graph(rng, n, e):
    src, dst = rng.integers(0, n, e), rng.integers(0, n, e)
    order = np.lexsort((src, dst))
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(indptr, dst + 1, 1)
    return src, dst, np.cumsum(indptr), src[order], order


def test_spmm_against_scipy_and_c():
    rng = np.random.default_rng(1)
    n, e = 200, 3000
    src, dst, indptr, indices, eids = _rand_graph(rng, n, e)
    nq = rng.integers(-127, 128, (n, 2, 24), dtype=np.int8)
    eq = rng.integers(-127, 128, (e, 2), dtype=np.int8)
    a = sp.csr_matrix((np.ones(e), indices, indptr), shape=(n, n))
    ref = (a @ nq.reshape(n, -1).astype(np.float64)).astype(np.float32) * np.float32(0.5)
    got = O.spmm_copy_u(indptr, indices, nq, np.float32(0.5))
    np.testing.assert_array_equal(got, ref)
    np.testing.assert_array_equal(got, C.spmm_copy_u(indptr, indices, nq, 0.5))
    for h in range(2):
        ah = sp.csr_matrix((eq[eids, h].astype(np.float64), indices, indptr), shape=(n, n))
        refh = (ah @ nq[:, h, :].astype(np.float64)).astype(np.float32) * np.float32(0.25)
        np.testing.assert_array_equal(O.spmm_u_mul_e(indptr, indices, eids, nq, eq, np.float32(0.25))[:, h], refh)
    np.testing.assert_array_equal(O.spmm_u_mul_e(indptr, indices, eids, nq, eq, np.float32(0.25)),
                                  C.spmm_u_mul_e(indptr, indices, eids, nq, eq, 0.25))
    inc = sp.csr_matrix((np.ones(e), (dst, np.arange(e))), shape=(n, e))
    np.testing.assert_array_equal(O.spmm_incidence(indptr, eids, eq, np.float32(2.0)),
                                  (inc @ eq.astype(np.float64)).astype(np.float32) * np.float32(2.0))
    np.testing.assert_array_equal(O.sddmm_dot(src, dst, nq, nq, np.float32(0.1), np.float32(0.3)),
                                  C.sddmm_dot(src, dst, nq, nq, 0.1, 0.3))


def test_sharded_scales_reduce_to_single_scale():
    rng = np.random.default_rng(2)
    n, e = 120, 2000
    _, _, indptr, indices, _ = _rand_graph(rng, n, e)
    nq = rng.integers(-3, 4, (n, 8), dtype=np.int8)      # small values: per-shard fp32 sums stay exact
    one = O.spmm_copy_u(indptr, indices, nq, np.float32(0.5))
    four = O.spmm_copy_u(indptr, indices, nq, np.full(4, 0.5, np.float32), shard_rows=30)
    np.testing.assert_array_equal(one, four)


def test_backward_gemm_linearity_and_transpose_identity():
    rng = np.random.default_rng(3)
    dy = rng.integers(-127, 128, (50, 12), dtype=np.int8)
    x = rng.integers(-127, 128, (50, 20), dtype=np.int8)
    w = rng.integers(-127, 128, (12, 20), dtype=np.int8)
    one = np.float32(1.0)
    # <dY, X W^T> = <dY W, X> = <dY^T X, W>
    lhs = np.sum(dy.astype(np.int64) * O.qgemm_acc_nt(x, w))
    assert lhs == np.sum(O.qgemm_backward_dx(dy, w, one, one).astype(np.int64) * x)
    assert lhs == np.sum(O.qgemm_backward_dw(dy, x, one, one).astype(np.int64) * w)
    np.testing.assert_array_equal(C.igemm_nt(x, w), O.qgemm_acc_nt(x, w))


def test_golden_file_regression():
    g = GOLD
    s = g["q_scale"][0]
    assert s == O.absmax_scale(g["q_x"])
    for mode, name in ((0, "trunc"), (1, "nearest"), (2, "stoch")):
        np.testing.assert_array_equal(O.quantize(g["q_x"], s, mode, seed=42, call=7), g[f"q_{name}"])
    y, aq, bq, *_ = O.qgemm_forward(g["gemm_a"], g["gemm_b"], sx=np.float32(0.5), sw=np.float32(0.5))
    np.testing.assert_array_equal(y, g["gemm_y"])
    np.testing.assert_array_equal(O.spmm_copy_u(g["g_indptr"], g["g_indices"], g["g_nq"], np.float32(0.02)),
                                  g["spmm_copy_u"])
    np.testing.assert_array_equal(
        O.spmm_u_mul_e(g["g_indptr"], g["g_indices"], g["g_eids"], g["g_nq"], g["g_eq"], np.float32(0.001)),
        g["spmm_u_mul_e"])


def test_edge_softmax_rows_sum_to_one():
    rng = np.random.default_rng(4)
    src, dst, indptr, indices, eids = _rand_graph(rng, 30, 400)
    z = rng.standard_normal((400, 3)).astype(np.float32)
    a = O.edge_softmax(indptr, eids, z)
    sums = np.zeros((30, 3))
    np.add.at(sums, dst, a)
    np.testing.assert_allclose(sums[np.diff(indptr) > 0], 1.0, rtol=1e-5)


# ----------------------------------------------------------------------------------------------------------------
# The oracle against outputs of the REFERENCE's own CUDA kernels (tests/golden/ref_fixtures*.npz, produced on a B200
# by tests/golden/make_ref_fixtures.py from the module oracle/build_ref.py compiles out of the reference's sources
# with the reference's flags).  The reference is built with --use_fast_math: its divisions are approximate and its
# a*s + b*t contracts into a fused multiply-add, so where such an operation is involved the comparison allows what
# that can change (stated per case); everything else must match bit for bit.
# ----------------------------------------------------------------------------------------------------------------
_REF_PATH = os.path.join(os.path.dirname(__file__), "golden", "ref_fixtures.npz")
_REF_SP_PATH = os.path.join(os.path.dirname(__file__), "golden", "ref_fixtures_cusparse.npz")
needs_ref = pytest.mark.skipif(not os.path.exists(_REF_PATH), reason="reference fixtures not generated")
needs_ref_sp = pytest.mark.skipif(not os.path.exists(_REF_SP_PATH), reason="reference cuSPARSE fixtures not generated")


def _ulps(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))


@needs_ref
def test_reference_get_scale_and_quantize():
    r = np.load(_REF_PATH)
    x, s_ref = r["q_x"], r["q_scale"][0]
    # max|x| / 127 with an approximate division: within 2 ulp of the IEEE quotient
    assert _ulps(s_ref, O.absmax_scale(x)).max() <= 2
    # power-of-two scale: the reciprocal is exact in either arithmetic -> every code, ties included, must match
    np.testing.assert_array_equal(O.quantize(x, np.float32(0.0625)), r["q_out_pow2"])
    np.testing.assert_array_equal(O.quantize(r["q_ties_x"], np.float32(0.0625)), r["q_ties_out"])   # half to even
    np.testing.assert_array_equal(C.quantize(r["q_ties_x"], 0.0625, 1), r["q_ties_out"])
    # natural scale: x * (1/s) with an approximate reciprocal may land on the other side of a .5 boundary
    q = O.quantize(x, s_ref).astype(np.int32)
    diff = np.abs(q - r["q_out"].astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3


@needs_ref
def test_reference_transpose_quant():
    r = np.load(_REF_PATH)
    for tag in ("a", "b"):
        x, s, out = r[f"tq_{tag}_x"], r[f"tq_{tag}_scale"][0], r[f"tq_{tag}_out"]
        mine = O.transpose_quant(x, s).reshape(out.shape).astype(np.int32)
        diff = np.abs(mine - out.astype(np.int32))
        assert diff.max() <= 1 and (diff != 0).mean() < 2e-3


@needs_ref
def test_reference_sddmm():
    r = np.load(_REF_PATH)
    src, dst = r["sd_src"], r["sd_dst"]
    for tag in ("h4d16", "h1d70", "h2d33"):
        u, v, su, sv = r[f"sd_{tag}_u"], r[f"sd_{tag}_v"], r[f"sd_{tag}_su"][0], r[f"sd_{tag}_sv"][0]
        mine = O.sddmm_dot(src, dst, u, v, su, sv)
        np.testing.assert_array_equal(mine, r[f"sd_{tag}_out"][..., 0])           # int32 dot, one fp32 multiply
        np.testing.assert_array_equal(C.sddmm_dot(src, dst, u, v, su, sv), r[f"sd_{tag}_out"][..., 0])
        assert _ulps(r[f"sd_{tag}_scale_out"][0], O.absmax_scale(mine)).max() <= 2
    u, v, su, sv = r["se_u"], r["se_v"], r["se_su"][0], r["se_sv"][0]
    np.testing.assert_array_equal(O.sddmm_elementwise("mul", src, dst, u, v, su, sv), r["se_mul_out"][..., 0])
    for op in ("add", "sub"):       # a*su + b*sv contracts into one FMA under fast-math: last-bit differences
        np.testing.assert_allclose(O.sddmm_elementwise(op, src, dst, u, v, su, sv), r[f"se_{op}_out"][..., 0],
                                   rtol=0, atol=2e-7 * 127 * 0.03)
    assert _ulps(O.sddmm_elementwise("div", src, dst, u, v, su, sv), r["se_div_out"][..., 0]).max() <= 4


@needs_ref
def test_reference_backward_gemms():
    r = np.load(_REF_PATH)
    for tag in ("a", "b"):
        dy, w, x = r[f"bg_{tag}_dy"], r[f"bg_{tag}_w"], r[f"bg_{tag}_x"]
        sdy, sw, sx = r[f"bg_{tag}_sdy"][0], r[f"bg_{tag}_sw"][0], r[f"bg_{tag}_sx"][0]
        np.testing.assert_array_equal(O.qgemm_backward_dx(dy, w, sdy, sw), r[f"bg_{tag}_dx"])
        np.testing.assert_array_equal(O.qgemm_backward_dw(dy, x, sdy, sx), r[f"bg_{tag}_dw"])


@needs_ref_sp
def test_reference_cusparse_spmm():
    """csr_SPMM and multi_cusparse_SPMM of the reference are cuSPARSE calls with fp32 compute type: the library
    accumulates (and applies alpha) in fp32 in an order of its own, the oracle sums exactly in integers and scales
    once.  Four values in five agree bit for bit, the rest within fp32 rounding: the bar is 1e-6 of the tensor's
    largest magnitude (measured: 9e-8), three orders below the 1e-3 the operator outputs are held to."""
    r = np.load(_REF_SP_PATH)
    indptr, indices, sc = r["sp_indptr"], r["sp_indices"], r["sp_scale"][0]
    mine = O.spmm_copy_u(indptr, indices, r["sp_nq"], sc)
    ref = r["sp_copy_u_out"]
    assert np.abs(mine - ref).max() <= 1e-6 * np.abs(ref).max()
    assert (mine == ref).mean() > 0.7
    eq = np.ascontiguousarray(r["sp_e_t"][:, 0, :].T)          # [nnz, H], already in slot order
    mine = O.spmm_u_mul_e(indptr, indices, None, r["sp_n3"], eq, sc)
    ref = r["sp_u_mul_e_out"]
    assert np.abs(mine - ref).max() <= 1e-6 * np.abs(ref).max()
    assert (mine == ref).mean() > 0.7
