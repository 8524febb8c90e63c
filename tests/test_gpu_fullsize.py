"""Parity at the sizes the benchmarks run at: the QLinear primitive at 232,965 x 602 -> 256, the SpMM / SDDMM
primitives on the 169,343-node / 1.17 M-edge graph, and the aggregation, weighted aggregation and dot SDDMM on the
232,965-node / 114.6 M-edge graph (whose hub rows have 100 K+ in-edges and go through the sliced-row path with
int32 atomics).  The small graphs are checked in full against the CPU oracle; the 114.6 M-edge graph is checked on a
row sample that always contains the ten longest rows, plus exact whole-graph integer checksums."""
import numpy as np
import pytest
import torch

from oracle import c_oracle as C
from oracle import tango_oracle as O

pytestmark = pytest.mark.gpu


def _s(v):
    return torch.tensor([float(v)], dtype=torch.float32, device="cuda")


# ------------------------------------------------------------------------------------------ QLinear primitive, full size
def test_qlinear_full_size_forward_dx_dw_bit_exact(cuda):
    from tango_b200 import kernels as K
    m, k, n = 232_965, 602, 256
    rng = np.random.default_rng(3)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = ((rng.random((n, k), dtype=np.float32) * 2 - 1) / np.float32(np.sqrt(k))).astype(np.float32)
    dy = rng.standard_normal((m, n), dtype=np.float32)
    xt, wt, dyt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(dy).cuda()
    sx, sw = K.cuda_kernels.get_scale(xt), K.cuda_kernels.get_scale(wt)
    assert sx.item() == O.absmax_scale(x) and sw.item() == O.absmax_scale(w)
    xq, wq = K.alloc_int8(xt.shape, "cuda"), K.alloc_int8(wt.shape, "cuda")
    y, sy = K.QGEMM_forward(xt, xq, sx, wt, wq, sw, None, True)       # truncating fused forward, output scale
    ry, rxq, rwq, rsx, rsw, rsy = O.qgemm_forward(x, w, reduce_out=True)
    np.testing.assert_array_equal(xq.cpu().numpy(), rxq)
    np.testing.assert_array_equal(wq.cpu().numpy(), rwq)
    np.testing.assert_array_equal(y.cpu().numpy(), ry)
    assert sy.item() == rsy
    del y, ry
    dyq, sdy = K.quantize(dyt)
    rdyq = C.quantize(dy, O.absmax_scale(dy), 1)
    assert sdy.item() == O.absmax_scale(dy)
    np.testing.assert_array_equal(dyq.cpu().numpy(), rdyq)
    dx, dw = K.QGEMM_backward(dyq, xq, wq, sdy, sx, sw)
    assert K.device_status() == 0
    np.testing.assert_array_equal(dw.cpu().numpy(), O.qgemm_backward_dw(rdyq, rxq, sdy.item(), rsx))
    np.testing.assert_array_equal(dx.cpu().numpy(), O.qgemm_backward_dx(rdyq, rwq, sdy.item(), rsw))


# ------------------------------------------------------------------------------------------ SpMM / SDDMM graph, full size
@pytest.fixture(scope="module")
def arxiv_like():
    import tango_b200 as T
    from tango_b200.graph import rmat_graph
    g = rmat_graph(169_343, 1_166_243, 20243, device="cuda")
    T.graph_preprocess(g)
    csc = [t.cpu().numpy().astype(np.int64) for t in g.adj_csc]
    csr = [t.cpu().numpy().astype(np.int64) for t in g.adj_csr]
    src, dst = [t.cpu().numpy().astype(np.int64) for t in g.coo]
    return g, csc, csr, src, dst


@pytest.mark.parametrize("f", [128, 256])
def test_spmm_sddmm_full_size_vs_oracle(cuda, arxiv_like, f):
    from tango_b200 import kernels as K
    g, csc, csr, src, dst = arxiv_like
    n, e = g.num_nodes(), g.num_edges()
    rng = np.random.default_rng(f)
    nq = rng.integers(-127, 128, (n, f), dtype=np.int8)
    eq = rng.integers(-127, 128, (e, 4), dtype=np.int8)
    nt, et = torch.from_numpy(nq).cuda(), torch.from_numpy(eq).cuda()
    sc = np.float32(0.0173)
    # copy-u, both directions
    np.testing.assert_array_equal(K.csr_SPMM(g, nt, _s(sc)).cpu().numpy(), C.spmm_copy_u(csc[0], csc[1], nq, sc))
    np.testing.assert_array_equal(K.csr_SPMM(g, nt, _s(sc), True).cpu().numpy(), C.spmm_copy_u(csr[0], csr[1], nq, sc))
    # per-head edge weights (4 heads), forward graph
    n3 = nq.reshape(n, 4, f // 4)
    out = K.spmm_u_mul_e_int8(g, nt.view(n, 4, f // 4), et, _s(sc))
    np.testing.assert_array_equal(out.cpu().numpy(), C.spmm_u_mul_e(csc[0], csc[1], csc[2], n3, eq, sc))
    out = K.spmm_u_mul_e_int8(g, nt.view(n, 4, f // 4), et, _s(sc), True)
    np.testing.assert_array_equal(out.cpu().numpy(), C.spmm_u_mul_e(csr[0], csr[1], csr[2], n3, eq, sc))
    # dot SDDMM with 1 and 4 heads
    for h in (1, 4):
        v3 = nq.reshape(n, h, f // h)
        got, so = K.mySDDMM_int8(g, "dot", nt.view(n, h, f // h), nt.view(n, h, f // h), _s(0.5), _s(0.25), True)
        ref = C.sddmm_dot(src, dst, v3, v3, 0.5, 0.25)
        np.testing.assert_array_equal(got.cpu().numpy()[..., 0], ref)
        assert so.item() == O.absmax_scale(ref)


def test_incidence_and_elementwise_full_size_vs_oracle(cuda, arxiv_like):
    from tango_b200 import kernels as K
    g, csc, csr, src, dst = arxiv_like
    n, e = g.num_nodes(), g.num_edges()
    rng = np.random.default_rng(9)
    for width in (4, 16, 32):
        zq = rng.integers(-127, 128, (e, width), dtype=np.int8)
        zt = torch.from_numpy(zq).cuda()
        np.testing.assert_array_equal(K.incidence_SPMM(g, zt, _s(0.031)).cpu().numpy(),
                                      O.spmm_incidence(csc[0], csc[2], zq, np.float32(0.031)))
        np.testing.assert_array_equal(K.incidence_SPMM(g, zt, _s(0.031), True).cpu().numpy(),
                                      O.spmm_incidence(csr[0], csr[2], zq, np.float32(0.031)))
    uq = rng.integers(-127, 128, (n, 1, 16), dtype=np.int8)
    ut = torch.from_numpy(uq).cuda()
    got, _ = K.mySDDMM_int8(g, "add", ut, ut, _s(0.02), _s(0.05), False)
    np.testing.assert_array_equal(got.cpu().numpy().reshape(e, 16),
                                  O.sddmm_elementwise("add", src, dst, uq, uq, np.float32(0.02), np.float32(0.05)))


# ------------------------------------------------------------------------------------------ the 114.6 M-edge graph
@pytest.fixture(scope="module")
def reddit_like():
    import tango_b200 as T
    from tango_b200.graph import rmat_graph
    g = rmat_graph(232_965, 114_615_892 - 232_965, 20245, device="cuda")
    T.graph_preprocess(g)              # default settings: the dense hub block is built for a graph of this size
    assert "csc" in g._hubs and g._hubs["csc"].density > 0.1
    indptr = g.adj_csc[0].cpu().numpy().astype(np.int64)
    deg = np.diff(indptr)
    rng = np.random.default_rng(5)
    rows = np.unique(np.concatenate([np.argsort(deg)[-10:], np.argsort(deg)[:5], rng.integers(0, g.num_nodes(), 150)]))
    return g, indptr, rows


def _row_slices(g, indptr, rows, reverse=False):
    bundle = g.adj_csr if reverse else g.adj_csc
    out = []
    for v in rows:
        b, e = int(indptr[v]), int(indptr[v + 1])
        out.append(bundle[1][b:e].cpu().numpy().astype(np.int64))
    return out


@pytest.mark.parametrize("hub", [True, False])
@pytest.mark.parametrize("f", [256, 41])
def test_aggregation_hub_rows_vs_oracle(cuda, reddit_like, f, hub):
    """F = 256 (layer 1) and F = 41 (layer 2, rows padded to 48 bytes): sampled rows -- the ten longest among them,
    up to 108 K in-edges -- equal the oracle's integer row sums times the scale, bit for bit; with the dense hub
    block on the tensor cores (the default for this graph) and with every edge gathered (sliced rows, int32 atomics)."""
    from tango_b200 import kernels as K
    g, indptr, rows = reddit_like
    hubs = g._hubs
    try:
        if not hub:
            g._hubs = {}
        _check_aggregation(g, indptr, rows, f)
    finally:
        g._hubs = hubs


def _check_aggregation(g, indptr, rows, f):
    from tango_b200 import kernels as K
    n = g.num_nodes()
    assert np.diff(indptr).max() > 100_000
    rng = np.random.default_rng(f)
    nq = rng.integers(-127, 128, (n, f), dtype=np.int8)
    nt = K.alloc_int8((n, f), "cuda")
    torch.as_strided(nt, (n, nt.stride(0)), (nt.stride(0), 1)).zero_()
    nt.copy_(torch.from_numpy(nq).cuda())
    sc = np.float32(0.0113)
    out = K.csr_SPMM(g, nt, _s(sc))
    got = out[torch.from_numpy(rows).cuda()].cpu().numpy()
    for i, cols in enumerate(_row_slices(g, indptr, rows)):
        acc = nq[cols].astype(np.int64).sum(0)
        np.testing.assert_array_equal(got[i], (acc.astype(np.float32) * sc).astype(np.float32))
    # whole-graph checksum: with scale 1 every output is the exact integer sum (|sum| < 2^24), and the column totals
    # over all rows must equal sum_u outdeg(u) * N_q[u, :]
    out1 = K.csr_SPMM(g, nt, _s(1.0))
    total = out1.double().sum(0).cpu().numpy()
    want = (g.out_degrees().cpu().numpy().astype(np.int64)[:, None] * nq.astype(np.int64)).sum(0)
    np.testing.assert_array_equal(total.astype(np.int64), want)


def test_weighted_aggregation_and_dot_sddmm_hub_rows_vs_oracle(cuda, reddit_like):
    """4 heads x 64: int8-weighted aggregation and the row-wise dot SDDMM on the sampled rows (hub rows included)."""
    from tango_b200 import kernels as K
    g, indptr, rows = reddit_like
    assert g._identity.get("csc")        # slot j of the CSC holds edge j: per-edge tensors are in slot order
    n, e, h, d = g.num_nodes(), g.num_edges(), 4, 64
    rng = np.random.default_rng(17)
    nq = rng.integers(-127, 128, (n, h, d), dtype=np.int8)
    vq = rng.integers(-127, 128, (n, h, d), dtype=np.int8)
    nt, vt = torch.from_numpy(nq).cuda(), torch.from_numpy(vq).cuda()
    gen = torch.Generator(device="cuda").manual_seed(3)
    et = torch.randint(-127, 128, (e, h), dtype=torch.int8, device="cuda", generator=gen)
    sc = np.float32(0.00071)
    out = K.spmm_u_mul_e_int8(g, nt, et, _s(sc))
    dot, _ = K.mySDDMM_int8(g, "dot", nt, vt, _s(0.5), _s(0.125), False)      # [E, H, 1], edge ids follow the CSC
    got = out[torch.from_numpy(rows).cuda()].cpu().numpy()
    for i, (v, cols) in enumerate(zip(rows, _row_slices(g, indptr, rows))):
        b, e1 = int(indptr[v]), int(indptr[v + 1])
        wts = et[b:e1].cpu().numpy().astype(np.int64)                         # CSC slot j holds edge j on this graph
        acc = (nq[cols].astype(np.int64) * wts[:, :, None]).sum(0)
        assert np.abs(acc).max() < 2 ** 31
        np.testing.assert_array_equal(got[i], (acc.astype(np.float32) * sc).astype(np.float32))
        dacc = np.einsum("ehd,hd->eh", nq[cols].astype(np.int64), vq[v].astype(np.int64))
        ref = (dacc.astype(np.float32) * np.float32(0.5 * 0.125)).astype(np.float32)
        np.testing.assert_array_equal(dot[b:e1, :, 0].cpu().numpy(), ref)
