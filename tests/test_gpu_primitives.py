"""Parity of every CUDA primitive against the CPU oracle, through the C ABI (ctypes) on a B200.

Integer paths (quantized bytes, int32 accumulators and therefore every dequantized fp32 value, which is a single
rounded product of an exact integer) must be bit-exact.
"""
import numpy as np
import pytest
import torch

from oracle import tango_oracle as O

pytestmark = pytest.mark.gpu


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def _scale_t(s):
    return torch.tensor([float(s)], dtype=torch.float32, device="cuda")


def _graph(n, e, seed, loops=True):
    from tango_b200.graph import rmat_graph
    # edge ids in generation order (not CSC order): the kernels must follow the edge_ids indirection
    return rmat_graph(n, e, seed, device="cuda", self_loops=loops, edge_order="append")


def _np_graph(g):
    csr = [t.cpu().numpy().astype(np.int64) for t in g.adj_csr]
    csc = [t.cpu().numpy().astype(np.int64) for t in g.adj_csc]
    src, dst = [t.cpu().numpy().astype(np.int64) for t in g.coo]
    return csr, csc, src, dst


# ------------------------------------------------------------------------------------------------ quantisation
@pytest.mark.parametrize("shape", [(1,), (7,), (4096,), (33, 41), (128, 602), (257, 256), (5, 3, 16), (1000, 4, 1)])
def test_absmax_scale(cuda, shape):
    from tango_b200 import kernels as K
    x = np.random.default_rng(1).standard_normal(shape).astype(np.float32)
    s = K.cuda_kernels.get_scale(_dev(x))
    assert s.cpu().numpy()[0] == O.absmax_scale(x)


def test_absmax_zero_and_empty(cuda):
    from tango_b200 import kernels as K
    assert K.cuda_kernels.get_scale(torch.zeros(100, device="cuda")).item() == 0.0
    assert K.cuda_kernels.get_scale(torch.zeros((0, 8), device="cuda")).item() == 0.0


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("shape,align", [((64, 64), 16), ((33, 41), 16), ((128, 602), 16), ((1000, 4, 1), 1),
                                         ((19, 3), 16), ((4099,), 16), ((37, 4), 1), ((50, 2, 24), 16)])
def test_quantize_bit_exact(cuda, mode, shape, align):
    from tango_b200 import kernels as K
    rng = np.random.default_rng(7)
    x = (rng.standard_normal(shape) * 3).astype(np.float32)
    s = O.absmax_scale(x)
    q, st = K.quantize(_dev(x), None, mode=mode, seed=1234, call=5, align=align)
    assert st.item() == s
    ref = O.quantize(x, s, mode, seed=1234, call=5)
    got = q.cpu().numpy()
    assert got.shape == ref.shape
    np.testing.assert_array_equal(got, ref)
    if q.dim() >= 2 and q.stride(0) != q[0].numel():   # padded storage: the pad bytes must be zero
        store = torch.as_strided(q, (q.shape[0], q.stride(0)), (q.stride(0), 1))
        assert int(store[:, q[0].numel():].abs().sum().item()) == 0


def test_quantize_zero_scale_and_given_scale(cuda):
    from tango_b200 import kernels as K
    q, s = K.quantize(torch.zeros((8, 16), device="cuda"))
    assert s.item() == 0 and int(q.abs().sum()) == 0
    x = np.linspace(-4, 4, 64, dtype=np.float32).reshape(4, 16)
    q, _ = K.quantize(_dev(x), _scale_t(0.01))           # saturates: clamp to +-127
    np.testing.assert_array_equal(q.cpu().numpy(), O.quantize(x, np.float32(0.01)))
    assert q.max().item() == 127 and q.min().item() == -127


def test_quantize_row_scale(cuda):
    from tango_b200 import kernels as K
    rng = np.random.default_rng(3)
    x = rng.standard_normal((100, 48)).astype(np.float32)
    rs = rng.random(100).astype(np.float32)
    xs = (x * rs[:, None]).astype(np.float32)
    s = K._get_scale(_dev(x), _dev(rs))
    assert s.item() == O.absmax_scale(xs)
    out = K.alloc_int8(x.shape, "cuda")
    K._quantize_into(out, _dev(x), s, 1, 0, 0, _dev(rs))
    np.testing.assert_array_equal(out.cpu().numpy(), O.quantize(xs, O.absmax_scale(xs)))


@pytest.mark.parametrize("shape", [(64, 602), (257, 41), (5, 7), (3, 5), (1000, 6), (33, 4099)])
def test_absmax_with_row_factors_on_unaligned_rows(cuda, shape):
    """Contiguous rows that do not start on 16-byte boundaries are read as one flat vector stream; vectors that
    straddle a row boundary must take each element's own row factor."""
    from tango_b200 import kernels as K
    rng = np.random.default_rng(shape[1])
    x = rng.standard_normal(shape).astype(np.float32)
    rs = (rng.random(shape[0]) * 10).astype(np.float32)
    rs[rng.integers(0, shape[0])] = 1000.0               # one row dominates: a wrong row factor shows immediately
    xs = (x * rs[:, None]).astype(np.float32)
    assert K._get_scale(_dev(x), _dev(rs)).item() == O.absmax_scale(xs)


def test_stochastic_rounding_is_unbiased_and_seeded(cuda):
    from tango_b200 import kernels as K
    x = torch.full((1 << 16,), 0.3, device="cuda")
    x[0] = 1.0                                          # scale = 1/127 -> 0.3 maps to 38.1
    a, _ = K.quantize(x, None, mode=2, seed=9, call=1)
    b, _ = K.quantize(x, None, mode=2, seed=9, call=1)
    c, _ = K.quantize(x, None, mode=2, seed=9, call=2)
    assert torch.equal(a, b) and not torch.equal(a, c)
    mean = a[1:].float().mean().item()
    assert abs(mean - 38.1) < 0.02
    assert set(a[1:].unique().tolist()) == {38, 39}


def test_stochastic_rounding_step_counter_survives_graph_replay(cuda):
    """The device-side step word is added (shifted by 32) to the call counter: equal to the oracle with that counter,
    and a captured CUDA graph that bumps the word draws new random numbers at every replay."""
    from tango_b200 import config, kernels as K
    rng = np.random.default_rng(8)
    x = rng.standard_normal((64, 41)).astype(np.float32)
    xd = _dev(x)
    s = O.absmax_scale(x)
    counter = torch.zeros(1, dtype=torch.int64, device="cuda")
    config.set_step_counter(counter)
    try:
        counter.fill_(3)
        q, _ = K.quantize(xd, None, mode=2, seed=77, call=5)
        np.testing.assert_array_equal(q.cpu().numpy(), O.quantize(x, s, 2, seed=77, call=5 + (3 << 32)))
        # graph: bump the word, then quantize; scalar arguments (call = 5) are frozen at capture time
        counter.zero_()
        st = _scale_t(s)
        out = K.alloc_int8(x.shape, "cuda")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            K._quantize_into(out, xd, st, 2, 77, 5)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            counter.add_(1)
            K._quantize_into(out, xd, st, 2, 77, 5)
        seen = []
        for k in range(1, 4):
            graph.replay()
            torch.cuda.synchronize()
            assert int(counter) == k
            got = out.cpu().numpy().copy()
            np.testing.assert_array_equal(got, O.quantize(x, s, 2, seed=77, call=5 + (k << 32)))
            seen.append(got)
        assert not np.array_equal(seen[0], seen[1]) and not np.array_equal(seen[1], seen[2])
    finally:
        config.set_step_counter(None)


def test_transpose_quant(cuda):
    from tango_b200 import kernels as K
    rng = np.random.default_rng(11)
    e = rng.random((1000, 4, 1)).astype(np.float32)
    s = O.absmax_scale(e)
    got = K.transpose_quant(_dev(e), _scale_t(s)).cpu().numpy()
    np.testing.assert_array_equal(got, O.transpose_quant(e, s))
    e2 = rng.standard_normal((77, 3, 5)).astype(np.float32)
    s2 = O.absmax_scale(e2)
    np.testing.assert_array_equal(K.transpose_quant(_dev(e2), _scale_t(s2)).cpu().numpy(), O.transpose_quant(e2, s2))


# ------------------------------------------------------------------------------------------------ SpMM
@pytest.mark.parametrize("f", [4, 16, 41, 128, 256, 602])
def test_spmm_copy_u(cuda, f):
    from tango_b200 import kernels as K
    g = _graph(500, 6000, 3)
    (csr, csc, src, dst) = _np_graph(g)
    rng = np.random.default_rng(f)
    nq = rng.integers(-127, 128, (500, f), dtype=np.int8)
    nq_t = K.alloc_int8((500, f), "cuda"); nq_t.copy_(_dev(nq))
    if nq_t.stride(0) != f:
        torch.as_strided(nq_t, (500, nq_t.stride(0) - f), (nq_t.stride(0), 1), f).zero_()
    s = np.float32(0.0371)
    for reverse, (indptr, indices, _) in ((False, csc), (True, csr)):
        out = K.csr_SPMM(g, nq_t, _scale_t(s), reverse).cpu().numpy()
        np.testing.assert_array_equal(out, O.spmm_copy_u(indptr, indices, nq, s))


def test_spmm_copy_u_unaligned_contiguous(cuda):
    """API-level input: contiguous int8 with a row width that is not a multiple of 4 or 16."""
    from tango_b200 import kernels as K
    g = _graph(300, 2500, 5)
    (_, csc, _, _) = _np_graph(g)
    nq = np.random.default_rng(0).integers(-127, 128, (300, 41), dtype=np.int8)
    out = K.csr_SPMM(g, _dev(nq), _scale_t(0.5)).cpu().numpy()
    np.testing.assert_array_equal(out, O.spmm_copy_u(csc[0], csc[1], nq, np.float32(0.5)))


def test_spmm_long_rows_use_units(cuda):
    """A star graph: one row far above the split threshold, the rest of degree 1 (plus empty rows)."""
    from tango_b200 import kernels as K
    from tango_b200.graph import Graph
    n = 20000
    src = torch.arange(1, n - 5, dtype=torch.int32)
    dst = torch.zeros_like(src)
    extra_s = torch.arange(0, 3000, dtype=torch.int32)
    extra_d = torch.full_like(extra_s, 7)
    g = Graph(torch.cat([src, extra_s, dst[:50]]), torch.cat([dst, extra_d, src[:50]]), n).to("cuda")
    sched = K._schedule(g, False)
    assert sched.n_heavy == 2 and sched.n_units >= 9      # node 0 (19994 in-edges) and node 7 (3000)
    (_, csc, _, _) = _np_graph(g)
    nq = np.random.default_rng(2).integers(-127, 128, (n, 64), dtype=np.int8)
    out = K.csr_SPMM(g, _dev(nq), _scale_t(0.25)).cpu().numpy()
    np.testing.assert_array_equal(out, O.spmm_copy_u(csc[0], csc[1], nq, np.float32(0.25)))
    out2 = K.csr_SPMM(g, _dev(nq), _scale_t(0.25)).cpu().numpy()      # scratch is re-zeroed per call
    np.testing.assert_array_equal(out, out2)


def test_spmm_fused_epilogue(cuda):
    from tango_b200 import kernels as K
    g = _graph(400, 5000, 8)
    (_, csc, _, _) = _np_graph(g)
    rng = np.random.default_rng(4)
    nq = rng.integers(-127, 128, (400, 32), dtype=np.int8)
    rs = rng.random(400).astype(np.float32)
    bias = rng.standard_normal(32).astype(np.float32)
    s = np.float32(0.01)
    amax = torch.zeros(1, device="cuda")
    out = K.csr_SPMM(g, _dev(nq), _scale_t(s), False, _dev(rs), _dev(bias), True, amax).cpu().numpy()
    ref = O.spmm_copy_u(csc[0], csc[1], nq, s)
    ref = np.maximum((ref * rs[:, None]).astype(np.float32) + bias[None, :], 0).astype(np.float32)
    np.testing.assert_array_equal(out, ref)
    assert amax.item() == O.absmax_scale(ref)


@pytest.mark.parametrize("h,d", [(4, 64), (4, 32), (1, 41), (2, 24), (8, 1), (3, 5)])
def test_spmm_u_mul_e(cuda, h, d):
    from tango_b200 import kernels as K
    g = _graph(300, 4000, 13)
    (csr, csc, src, dst) = _np_graph(g)
    E = g.num_edges()
    rng = np.random.default_rng(h * 100 + d)
    nq = rng.integers(-127, 128, (300, h, d), dtype=np.int8)
    eq = rng.integers(-127, 128, (E, h), dtype=np.int8)
    nq_t = K.alloc_int8((300, h, d), "cuda"); nq_t.copy_(_dev(nq))
    ld = nq_t.stride(0)
    if ld != h * d:
        torch.as_strided(nq_t, (300, ld - h * d), (ld, 1), h * d).zero_()
    s = np.float32(0.003)
    for reverse, (indptr, indices, eids) in ((False, csc), (True, csr)):
        out = K.spmm_u_mul_e_int8(g, nq_t, _dev(eq), _scale_t(s), reverse).cpu().numpy()
        np.testing.assert_array_equal(out, O.spmm_u_mul_e(indptr, indices, eids, nq, eq, s))
    # reference-shaped call: E_T [H,1,E] as produced by transpose_quant
    e_t = _dev(np.ascontiguousarray(eq.T.reshape(h, 1, E)))
    out = K.multi_cusparse_SPMM(g, nq_t, e_t, _scale_t(s)).cpu().numpy()
    np.testing.assert_array_equal(out, O.spmm_u_mul_e(csc[0], csc[1], csc[2], nq, eq, s))


@pytest.mark.parametrize("dim", [1, 4, 16, 32])
def test_incidence_spmm(cuda, dim):
    from tango_b200 import kernels as K
    g = _graph(300, 4000, 17)
    (csr, csc, src, dst) = _np_graph(g)
    E = g.num_edges()
    zq = np.random.default_rng(dim).integers(-127, 128, (E, dim), dtype=np.int8)
    s = np.float32(0.02)
    out_in = K.incidence_SPMM(g, _dev(zq), _scale_t(s)).cpu().numpy()
    out_out = K.incidence_SPMM(g, _dev(zq), _scale_t(s), True).cpu().numpy()
    np.testing.assert_array_equal(out_in, O.spmm_incidence(csc[0], csc[2], zq, s))
    np.testing.assert_array_equal(out_out, O.spmm_incidence(csr[0], csr[2], zq, s))
    # the same sums straight from the definition: node v collects the edges whose dst (src) is v
    acc = np.zeros((300, dim), dtype=np.int64)
    np.add.at(acc, dst, zq.astype(np.int64))
    np.testing.assert_array_equal(out_in, (acc.astype(np.float32) * s).astype(np.float32))
    # reference-shaped native call with explicit COO (node, edge id) pairs
    inc = g.inc_in
    out = torch.empty((300, dim), device="cuda")
    K.cuda_kernels.incidence_SPMM(out, inc[0], inc[1], _dev(zq), _scale_t(s))
    np.testing.assert_array_equal(out.cpu().numpy(), out_in)


@pytest.mark.parametrize("dim", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("star", [False, True])
def test_incidence_spmm_contiguous_rows(cuda, dim, star):
    """Edges numbered in CSC order: the in-edge sums stream contiguous byte ranges (aligned 128-bit loads, ragged
    head and tail, hub rows cut into slices); must equal the oracle and the indirect (edge_ids) kernel bit for bit."""
    import tango_b200 as T
    from tango_b200 import kernels as K
    from tango_b200.graph import Graph, rmat_graph
    if star:
        n = 3000
        src = torch.cat([torch.arange(n).repeat(10), torch.arange(n)])
        dst = torch.cat([torch.zeros(10 * n, dtype=torch.long), (torch.arange(n) * 7 + 1) % n])
        perm = torch.argsort(dst * n + src, stable=True)
        g = Graph(src[perm], dst[perm], n).to("cuda")
    else:
        n = 700
        g = rmat_graph(n, 9000, 43, device="cuda", edge_order="dst")
    T.graph_preprocess(g)
    assert K._bundle(g, False)[2] is None                    # identity numbering detected
    (csr, csc, src_np, dst_np) = _np_graph(g)
    E = g.num_edges()
    zq = np.random.default_rng(dim).integers(-127, 128, (E, dim), dtype=np.int8)
    s = np.float32(0.02)
    out_in = K.incidence_SPMM(g, _dev(zq), _scale_t(s)).cpu().numpy()
    np.testing.assert_array_equal(out_in, O.spmm_incidence(csc[0], csc[2], zq, s))
    out_out = K.incidence_SPMM(g, _dev(zq), _scale_t(s), True).cpu().numpy()
    np.testing.assert_array_equal(out_out, O.spmm_incidence(csr[0], csr[2], zq, s))
    # the indirect kernel on the same data (explicit edge ids)
    out2 = torch.empty((n, dim), device="cuda")
    K._incidence_spmm(out2, g.adj_csc[0], g.adj_csc[2], _dev(zq), _scale_t(s), K._schedule(g, False))
    np.testing.assert_array_equal(out2.cpu().numpy(), out_in)


def test_spmm_segmented_per_shard_scales(cuda):
    """Row-partitioned form: nseg segments per row, one scale per source shard."""
    from tango_b200 import kernels as K
    from tango_b200.graph import RowPartition
    g = _graph(1000, 20000, 19)
    (_, csc, _, _) = _np_graph(g)
    world = 4
    nq = np.random.default_rng(5).integers(-127, 128, (1000, 64), dtype=np.int8)
    scales = np.array([0.01, 0.02, 0.005, 0.04], dtype=np.float32)
    ref = O.spmm_copy_u(csc[0], csc[1], nq, scales, shard_rows=250)
    for rank in range(world):
        part = RowPartition(g.adj_csc[0], g.adj_csc[1], None, 1000, rank, world)
        out = torch.empty((part.n_local, 64), device="cuda")
        K._csr_spmm(out, part.indptr, part.indices, _dev(nq), _dev(scales), part.schedule, world)
        np.testing.assert_array_equal(out.cpu().numpy(), ref[part.r0:part.r1])


# ------------------------------------------------------------------------------------------------ SDDMM
@pytest.mark.parametrize("h,d", [(1, 128), (4, 64), (4, 32), (1, 41), (2, 24), (3, 5), (1, 256)])
def test_sddmm_dot(cuda, h, d):
    from tango_b200 import kernels as K
    g = _graph(300, 4000, 23)
    (_, _, src, dst) = _np_graph(g)
    rng = np.random.default_rng(d)
    uq = rng.integers(-127, 128, (300, h, d), dtype=np.int8)
    vq = rng.integers(-127, 128, (300, h, d), dtype=np.int8)
    u_t = K.alloc_int8(uq.shape, "cuda"); u_t.copy_(_dev(uq))
    v_t = K.alloc_int8(vq.shape, "cuda"); v_t.copy_(_dev(vq))
    for t in (u_t, v_t):
        if t.stride(0) != h * d:
            torch.as_strided(t, (300, t.stride(0) - h * d), (t.stride(0), 1), h * d).zero_()
    su, sv = np.float32(0.01), np.float32(0.03)
    out, sc = K.mySDDMM_int8(g, "dot", u_t, v_t, _scale_t(su), _scale_t(sv), True)
    ref = O.sddmm_dot(src, dst, uq, vq, su, sv)
    assert out.shape == (g.num_edges(), h, 1)
    np.testing.assert_array_equal(out.cpu().numpy()[..., 0], ref)
    assert sc.item() == O.absmax_scale(ref)
    out_r, _ = K.mySDDMM_int8(g, "dot", u_t, v_t, _scale_t(su), _scale_t(sv), False, reverse=True)
    np.testing.assert_array_equal(out_r.cpu().numpy()[..., 0], O.sddmm_dot(dst, src, uq, vq, su, sv))


@pytest.mark.parametrize("h,d,order", [(4, 64, "dst"), (1, 41, "append"), (4, 16, "append"), (8, 4, "dst")])
def test_sddmm_dot_rows_matches_endpoint_kernel(cuda, h, d, order):
    """The row-wise dot kernel (fixed operand in registers, long rows cut into slices) against the endpoint-list
    kernel and the oracle, on a graph with a 30 000-edge hub row and on an arbitrarily numbered R-MAT graph."""
    import tango_b200 as T
    from tango_b200 import kernels as K
    from tango_b200.graph import Graph, rmat_graph
    if order == "dst":
        n = 3000
        src = torch.cat([torch.arange(n).repeat(10), torch.arange(n)])
        dst = torch.cat([torch.zeros(10 * n, dtype=torch.long), (torch.arange(n) * 7 + 1) % n])
        perm = torch.argsort(dst * n + src, stable=True)
        g = Graph(src[perm], dst[perm], n).to("cuda")
    else:
        n = 500
        g = rmat_graph(n, 9000, 41, device="cuda", edge_order="append")
    T.graph_preprocess(g)
    (_, _, src_np, dst_np) = _np_graph(g)
    rng = np.random.default_rng(h * 100 + d)
    uq = rng.integers(-127, 128, (n, h, d), dtype=np.int8)
    vq = rng.integers(-127, 128, (n, h, d), dtype=np.int8)
    u_t = K.alloc_int8(uq.shape, "cuda"); u_t.zero_(); u_t.copy_(_dev(uq))
    v_t = K.alloc_int8(vq.shape, "cuda"); v_t.zero_(); v_t.copy_(_dev(vq))
    for t in (u_t, v_t):
        if t.stride(0) != h * d:
            torch.as_strided(t, (n, t.stride(0) - h * d), (t.stride(0), 1), h * d).zero_()
    su, sv = _scale_t(np.float32(0.02)), _scale_t(np.float32(0.005))
    for reverse in (False, True):
        out = torch.empty((g.num_edges(), h, 1), device="cuda")
        sc = torch.zeros(1, device="cuda")
        indptr, indices, edge_ids = K._bundle(g, reverse)
        assert K._sddmm_dot_rows(out, sc, indptr, indices, edge_ids, u_t, v_t, su, sv, K._schedule(g, reverse))
        s_np, d_np = (dst_np, src_np) if reverse else (src_np, dst_np)
        ref = O.sddmm_dot(s_np, d_np, uq, vq, np.float32(0.02), np.float32(0.005))
        np.testing.assert_array_equal(out.cpu().numpy()[..., 0], ref)
        assert sc.item() == O.absmax_scale(ref)
        # the endpoint-list entry point on the same operands
        out2 = torch.empty_like(out)
        s_t, d_t = g.coo[::-1] if reverse else g.coo
        K.cuda_kernels.mySDDMM_int8("dot", out2, torch.Tensor(), s_t, d_t, u_t, v_t, su, sv)
        assert torch.equal(out, out2)
        # and the public wrapper, whichever of the two kernels it picks for this graph
        out3, sc3 = K.mySDDMM_int8(g, "dot", u_t, v_t, su, sv, True, reverse=reverse)
        assert torch.equal(out, out3) and sc3.item() == sc.item()


def test_sddmm_recipe_fixture(cuda):
    """The 3-node / 4-edge input recipe the reference keeps under #ifdef TEST (cuda/src/SDDMM.cu:230-257)."""
    from tango_b200 import kernels as K
    from tango_b200.graph import Graph
    for dim in (16, 64, 100):
        src, dst, u, v, su, sv = O.recipe_sddmm_inputs(dim)
        g = Graph(torch.from_numpy(src), torch.from_numpy(dst), 3).to("cuda")
        out, _ = K.mySDDMM_int8(g, "add", _dev(u), _dev(v), _scale_t(su), _scale_t(sv), False)
        np.testing.assert_array_equal(out.cpu().numpy().reshape(4, -1), O.sddmm_elementwise("add", src, dst, u, v, su, sv))
        out, _ = K.mySDDMM_int8(g, "dot", _dev(u), _dev(v), _scale_t(su), _scale_t(sv), False)
        np.testing.assert_array_equal(out.cpu().numpy().reshape(4, -1), O.sddmm_dot(src, dst, u, v, su, sv))


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("shape", [(4, 1), (1, 16), (3, 5), (1, 41)])
def test_sddmm_elementwise(cuda, op, shape):
    from tango_b200 import kernels as K
    g = _graph(300, 4000, 29)
    (_, _, src, dst) = _np_graph(g)
    rng = np.random.default_rng(1)
    uq = rng.integers(-127, 128, (300,) + shape, dtype=np.int8)
    vq = rng.integers(1, 128, (300,) + shape, dtype=np.int8)        # non-zero divisor
    su, sv = np.float32(0.01), np.float32(0.03)
    out, sc = K.mySDDMM_int8(g, op, _dev(uq), _dev(vq), _scale_t(su), _scale_t(sv), True)
    ref = O.sddmm_elementwise(op, src, dst, uq, vq, su, sv)
    np.testing.assert_array_equal(out.cpu().numpy().reshape(ref.shape), ref)
    assert sc.item() == O.absmax_scale(ref)


def test_gat_edge_softmax(cuda):
    from tango_b200 import kernels as K
    g = _graph(200, 3000, 31)
    (_, csc, src, dst) = _np_graph(g)
    rng = np.random.default_rng(2)
    el = rng.integers(-127, 128, (200, 4), dtype=np.int8)
    er = rng.integers(-127, 128, (200, 4), dtype=np.int8)
    sl, sr = np.float32(0.02), np.float32(0.015)
    a, sa = K.gat_edge_softmax(g, _dev(el), _dev(er), _scale_t(sl), _scale_t(sr), 0.2, want_scale=True)
    assert sa.item() == (a.max() / 127).item()               # the epilogue's scale is the quantizer's scale
    a = a.cpu().numpy()
    z = O.leaky_relu(O.sddmm_elementwise("add", src, dst, el, er, sl, sr), 0.2)
    ref = O.edge_softmax(csc[0], csc[2], z)
    np.testing.assert_allclose(a, ref, rtol=1e-4, atol=1e-6)   # fp32 exp: tolerance, not bit-exact
    sums = np.zeros((200, 4)); np.add.at(sums, dst, a)
    np.testing.assert_allclose(sums, 1.0, rtol=1e-5)


@pytest.mark.parametrize("heads,order", [(4, "dst"), (4, "append"), (1, "dst"), (3, "append"), (8, "dst")])
def test_edge_softmax_plain_scores(cuda, heads, order):
    """Plain fp32 edge softmax (HGT's use) against the oracle, forward and gradient, with and without the edge-id
    indirection, incl. a destination with tens of thousands of incoming edges (CTA-per-row path)."""
    import tango_b200 as T
    from tango_b200 import kernels as K
    from tango_b200.graph import Graph, rmat_graph
    if order == "dst" and heads == 4:
        n = 3000                                             # star: node 0 receives an edge from everybody, 10 times
        src = torch.cat([torch.arange(n).repeat(10), torch.arange(n)])
        dst = torch.cat([torch.zeros(10 * n, dtype=torch.long), (torch.arange(n) * 7 + 1) % n])
        g = Graph(src, dst, n).to("cuda")
    else:
        g = rmat_graph(400, 5000, 37, device="cuda", edge_order=order)
    T.graph_preprocess(g)
    (_, csc, src_np, dst_np) = _np_graph(g)
    e = g.num_edges()
    rng = np.random.default_rng(heads)
    z = (rng.standard_normal((e, heads)) * 3).astype(np.float32)
    zmul = 0.35
    a, sa = K.edge_softmax_fwd(g, _dev(z).view(e, heads, 1), zmul, want_scale=True)
    assert a.shape == (e, heads, 1) and sa.item() == K.cuda_kernels.get_scale(a).item()
    ref = O.edge_softmax(csc[0], csc[2], (z * np.float32(zmul)).astype(np.float32))
    np.testing.assert_allclose(a.cpu().numpy().reshape(e, heads), ref, rtol=1e-4, atol=1e-7)
    # gradient against autograd of the same formula
    da = torch.from_numpy(rng.standard_normal((e, heads)).astype(np.float32)).cuda()
    dz, sdz = K.edge_softmax_bwd(g, a, da.view(e, heads, 1), zmul, want_scale=True)
    assert sdz.item() == K.cuda_kernels.get_scale(dz).item()
    dz = dz.reshape(e, heads)
    zt = _dev(z).requires_grad_(True)
    dstl = torch.from_numpy(dst_np).long().cuda()
    ex = torch.exp(zt * zmul - 2.0)
    ssum = torch.zeros(g.num_nodes(), heads, device="cuda").index_add_(0, dstl, ex)
    (ex / ssum[dstl] * da).sum().backward()
    assert (dz - zt.grad).abs().max() < 1e-4 * max(1.0, zt.grad.abs().max().item())


# ------------------------------------------------------------------------------------------------ empty inputs
def test_empty_graph_and_rows(cuda):
    from tango_b200 import kernels as K
    from tango_b200.graph import Graph
    g = Graph(torch.zeros(0, dtype=torch.int32), torch.zeros(0, dtype=torch.int32), 10).to("cuda")
    nq = torch.ones((10, 16), dtype=torch.int8, device="cuda")
    out = K.csr_SPMM(g, nq, _scale_t(1.0))
    assert out.shape == (10, 16) and float(out.abs().sum()) == 0.0
    o, _ = K.mySDDMM_int8(g, "dot", nq, nq, _scale_t(1.0), _scale_t(1.0), False)
    assert o.shape == (0, 1)


def test_csc_numbered_graph_skips_edge_id_indirection(cuda):
    """With edges numbered in CSC order the wrappers pass no edge_ids; results must match the indirect path."""
    from tango_b200 import kernels as K
    from tango_b200.graph import rmat_graph
    g = rmat_graph(300, 4000, 13, device="cuda")            # edge_order="dst"
    assert g.adj_csc is not None and g._identity["csc"] and K._bundle(g, False)[2] is None
    (csr, csc, src, dst) = _np_graph(g)
    np.testing.assert_array_equal(csc[2], np.arange(g.num_edges()))
    rng = np.random.default_rng(3)
    nq = rng.integers(-127, 128, (300, 4, 16), dtype=np.int8)
    eq = rng.integers(-127, 128, (g.num_edges(), 4), dtype=np.int8)
    s = np.float32(0.01)
    for reverse, (indptr, indices, eids) in ((False, csc), (True, csr)):
        out = K.spmm_u_mul_e_int8(g, _dev(nq), _dev(eq), _scale_t(s), reverse).cpu().numpy()
        np.testing.assert_array_equal(out, O.spmm_u_mul_e(indptr, indices, eids, nq, eq, s))
    np.testing.assert_array_equal(K.incidence_SPMM(g, _dev(eq), _scale_t(s)).cpu().numpy(),
                                  O.spmm_incidence(csc[0], csc[2], eq, s))


def test_row_gather_probe_runs_and_validates(cuda):
    """The benchmark's L2 row-gather probe lives in a library of its own (it is not part of the product ABI)."""
    import ctypes
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    probe = ctypes.CDLL(os.path.join(root, "tango_b200", "lib", "libtango_bench_probe.so")).bench_probe_row_gather
    probe.restype = ctypes.c_int64
    probe.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                      ctypes.c_void_p, ctypes.c_void_p]
    table = torch.ones((1000, 256), dtype=torch.int8, device="cuda")
    sink = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    nbytes = probe(table.data_ptr(), 1000, 256, 3, 8, 256, sink.data_ptr(), st)
    torch.cuda.synchronize()
    assert nbytes == 148 * 8 * 256 * 3 * 8 * 16 and int(sink) == 0
    assert probe(table.data_ptr(), 1000, 48, 3, 8, 256, sink.data_ptr(), st) == -1     # not a power of two
    assert probe(None, 1000, 256, 3, 8, 256, sink.data_ptr(), st) == -1



@pytest.mark.parametrize("f", [256, 41, 64])
@pytest.mark.parametrize("reverse", [False, True])
def test_copy_u_with_dense_hub_block_is_bit_identical(cuda, f, reverse):
    """Aggregation with the dense hub region multiplied on the tensor cores (forced here on a small graph: all tiles
    of the top 256 x 256 corner, then -- hub_block=-1 below -- a density-selected staircase) against the oracle and
    against the gather-only path: same bits."""
    import tango_b200 as T
    from tango_b200 import kernels as K
    from tango_b200.graph import rmat_graph
    g = rmat_graph(6000, 400_000, 41, device="cuda")
    T.graph_preprocess(g, hub_block=256)
    key = "csr" if reverse else "csc"
    assert key in g._hubs and g._hubs[key].n_block_edges > 0
    n = g.num_nodes()
    rng = np.random.default_rng(f)
    nq = rng.integers(-127, 128, (n, f), dtype=np.int8)
    nt = K.alloc_int8((n, f), "cuda")
    torch.as_strided(nt, (n, nt.stride(0)), (nt.stride(0), 1)).zero_()
    nt.copy_(torch.from_numpy(nq).cuda())
    sc = np.float32(0.0137)
    bias = torch.from_numpy(rng.standard_normal(f).astype(np.float32)).cuda()
    rs = torch.from_numpy(rng.random(n).astype(np.float32)).cuda()
    amax = torch.zeros(1, device="cuda")
    got = K.csr_SPMM(g, nt, _scale_t(sc), reverse, rs, bias, True, amax)
    assert K.device_status() == 0
    bundle = g.adj_csr if reverse else g.adj_csc
    ip, idx = [t.cpu().numpy().astype(np.int64) for t in bundle[:2]]
    ref = O.spmm_copy_u(ip, idx, nq, sc)
    ref = np.maximum((ref * rs.cpu().numpy()[:, None]).astype(np.float32) + bias.cpu().numpy()[None, :], 0).astype(np.float32)
    np.testing.assert_array_equal(got.cpu().numpy(), ref)
    assert amax.item() == O.absmax_scale(ref)
    T.graph_preprocess(g, hub_block=0)
    assert not g._hubs
    plain = K.csr_SPMM(g, nt, _scale_t(sc), reverse, rs, bias, True)
    assert torch.equal(plain, got)
    # a staircase chosen by density (several row tiles with different extents, several work items per row tile)
    from tango_b200.graph import HubBlock
    ipt, idt, _ = g.adj_csr if reverse else g.adj_csc
    hub = HubBlock(ipt, idt, n, 4096, 4096, 0.02)
    assert hub.ok and hub.kend.numel() > 2 and int(hub.kend.min()) < int(hub.kend.max())
    g._hubs = {key: hub}
    stair = K.csr_SPMM(g, nt, _scale_t(sc), reverse, rs, bias, True)
    assert K.device_status() == 0 and torch.equal(stair, got)
