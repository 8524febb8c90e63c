"""tcgen05 int8 GEMMs (forward, dX, dW) against the CPU oracle: int32 accumulators and the dequantized fp32 values
must be bit-exact, for aligned, ragged and tiny shapes."""
import numpy as np
import pytest
import torch

from oracle import tango_oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [  # (M, N, K)
    (128, 16, 128), (128, 256, 128), (256, 64, 256), (300, 41, 256), (1000, 256, 602), (513, 16, 500),
    (19, 3, 16), (4096, 256, 608), (777, 602, 256), (128, 48, 32), (1, 16, 16), (200, 300, 100),
]


def _pad_copy(a):
    from tango_b200 import kernels as K
    t = K.alloc_int8(a.shape, "cuda")
    ld = t.stride(0)
    torch.as_strided(t, (a.shape[0], ld), (ld, 1)).zero_()
    t.copy_(torch.from_numpy(a).cuda())
    return t


def _s(v):
    return torch.tensor([float(v)], dtype=torch.float32, device="cuda")


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_qgemm_nt(cuda, m, n, k):
    from tango_b200 import kernels as K
    rng = np.random.default_rng(m + n + k)
    xq = rng.integers(-127, 128, (m, k), dtype=np.int8)
    wq = rng.integers(-127, 128, (n, k), dtype=np.int8)
    bias = rng.standard_normal(n).astype(np.float32)
    sx, sw = np.float32(0.013), np.float32(0.0021)
    y = torch.empty((m, n), device="cuda")
    sy = torch.zeros(1, device="cuda")
    K._qgemm_nt(y, _pad_copy(xq), _pad_copy(wq), _s(sx), _s(sw), torch.from_numpy(bias).cuda(), sy)
    assert K.device_status() == 0
    ref = O.dequant(O.qgemm_acc_nt(xq, wq), sx, sw, bias)
    np.testing.assert_array_equal(y.cpu().numpy(), ref)
    assert sy.item() == O.absmax_scale(ref)


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_qgemm_dx(cuda, m, n, k):
    from tango_b200 import kernels as K
    rng = np.random.default_rng(m * 3 + n + k)
    dyq = rng.integers(-127, 128, (m, n), dtype=np.int8)
    wq = rng.integers(-127, 128, (n, k), dtype=np.int8)
    s1, s2 = np.float32(0.5), np.float32(0.25)
    dx = torch.empty((m, k), device="cuda")
    K.cuda_kernels.QGEMM_backward_gradX(dx, _pad_copy(dyq), _pad_copy(wq), _s(s1), _s(s2))
    assert K.device_status() == 0
    np.testing.assert_array_equal(dx.cpu().numpy(), O.qgemm_backward_dx(dyq, wq, s1, s2))


@pytest.mark.parametrize("m,n,k", SHAPES + [(50000, 256, 602), (20000, 41, 256)])
def test_qgemm_dw(cuda, m, n, k):
    from tango_b200 import kernels as K
    rng = np.random.default_rng(m * 5 + n + k)
    dyq = rng.integers(-127, 128, (m, n), dtype=np.int8)
    xq = rng.integers(-127, 128, (m, k), dtype=np.int8)
    s1, s2 = np.float32(0.5), np.float32(0.125)
    dw = torch.empty((n, k), device="cuda")
    K.cuda_kernels.QGEMM_backward_gradW(dw, _pad_copy(dyq), _pad_copy(xq), _s(s1), _s(s2))
    assert K.device_status() == 0
    np.testing.assert_array_equal(dw.cpu().numpy(), O.qgemm_backward_dw(dyq, xq, s1, s2))


def test_gemm_recipe_fixture(cuda):
    """Input recipe of the reference's #ifdef TEST main (cuda/src/QGEMM_forward.cu:162-210): A, B in [-8, 7], scales
    0.5; the fused forward quantizes by truncation and must reproduce the oracle exactly."""
    from tango_b200 import kernels as K
    m, n, k = 512, 256, 256
    a, b, sa, sb = O.recipe_gemm_inputs(m, n, k)
    x, w = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    xq, wq = K.alloc_int8(x.shape, "cuda"), K.alloc_int8(w.shape, "cuda")
    y = K.QGEMM_forward(x, xq, _s(sa), w, wq, _s(sb))
    ref, rxq, rwq, *_ = O.qgemm_forward(a, b, sx=sa, sw=sb)
    np.testing.assert_array_equal(xq.cpu().numpy(), rxq)
    np.testing.assert_array_equal(wq.cpu().numpy(), rwq)
    np.testing.assert_array_equal(y.cpu().numpy(), ref)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_fused_forward_modes(cuda, mode):
    from tango_b200 import kernels as K
    rng = np.random.default_rng(mode)
    x = rng.standard_normal((700, 602)).astype(np.float32)
    w = (rng.random((256, 602)).astype(np.float32) - 0.5) * 0.08
    b = rng.standard_normal(256).astype(np.float32)
    ref, rxq, rwq, sx, sw, sy = O.qgemm_forward(x, w, b, mode=mode, reduce_out=True, seed=77, call=3)
    xt, wt = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    xq, wq = K.alloc_int8(xt.shape, "cuda"), K.alloc_int8(wt.shape, "cuda")
    y, s_out = K.QGEMM_forward(xt, xq, K.cuda_kernels.get_scale(xt), wt, wq, K.cuda_kernels.get_scale(wt),
                               torch.from_numpy(b).cuda(), True, mode=mode, seed=77, call=3)
    np.testing.assert_array_equal(xq.cpu().numpy(), rxq)
    np.testing.assert_array_equal(wq.cpu().numpy(), rwq)
    np.testing.assert_array_equal(y.cpu().numpy(), ref)
    assert s_out.item() == sy


def test_generic_qgemm_aliases(cuda):
    from tango_b200 import kernels as K
    rng = np.random.default_rng(0)
    a = rng.standard_normal((300, 64)).astype(np.float32)
    b = rng.standard_normal((48, 64)).astype(np.float32)
    sa, sb = O.absmax_scale(a), O.absmax_scale(b)
    aq, bq = O.quantize(a, sa), O.quantize(b, sb)
    got = K.cuda_kernels.QgemmNT(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()).cpu().numpy()
    np.testing.assert_array_equal(got, O.dequant(O.qgemm_acc_nt(aq, bq), sa, sb))
    rel = np.abs(got - a @ b.T).max() / np.abs(a @ b.T).max()
    assert rel < 0.05
