"""tango_qgemm_dw_noalloc: the weight-gradient GEMM for callers that cannot allocate device memory (hosts that
own all of it through their own pool, or loops that cannot afford cudaMalloc's device-wide synchronisation).  Its
scratch is a fixed array inside the library, shared by every call, so the test calls it twice in a row with different
inputs -- the second call must not see the first call's partial sums -- and compares each result bit-for-bit with
the regular entry point, which works in caller-provided scratch.  Collected last on purpose."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _padded(a):
    from tango_b200 import kernels as K
    t = K.alloc_int8(a.shape, "cuda")
    ld = t.stride(0)
    torch.as_strided(t, (a.shape[0], ld), (ld, 1)).zero_()
    t.copy_(torch.from_numpy(a).cuda())
    return t


def _run_both(m, n, k, seed):
    from tango_b200 import _lib
    L = _lib.lib
    rng = np.random.default_rng(seed)
    dyq = _padded(rng.integers(-127, 128, (m, n), dtype=np.int8))
    xq = _padded(rng.integers(-127, 128, (m, k), dtype=np.int8))
    s1 = torch.tensor([0.5], device="cuda")
    s2 = torch.tensor([0.03125], device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    ref = torch.empty((n, k), device="cuda")
    nbytes = L.tango_qgemm_dw_workspace_bytes(n, k)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    rc = L.tango_qgemm_dw(dyq.data_ptr(), dyq.stride(0), xq.data_ptr(), xq.stride(0), m, n, k, s1.data_ptr(),
                          s2.data_ptr(), ref.data_ptr(), k, ws.data_ptr(), nbytes, status.data_ptr(), stream)
    assert rc == 0
    got = torch.full((n, k), float("nan"), device="cuda")
    rc = L.tango_qgemm_dw_noalloc(dyq.data_ptr(), dyq.stride(0), xq.data_ptr(), xq.stride(0), m, n, k, s1.data_ptr(),
                                  s2.data_ptr(), got.data_ptr(), k, status.data_ptr(), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return got.cpu().numpy(), ref.cpu().numpy()


def test_noalloc_dw_matches_regular_entry_twice_in_a_row(cuda):
    got, ref = _run_both(30000, 256, 602, seed=1)
    np.testing.assert_array_equal(got, ref)
    assert np.abs(ref).max() > 0
    # second call, smaller problem with other data: stale partial sums of the first call must not leak in
    got2, ref2 = _run_both(5000, 41, 256, seed=2)
    np.testing.assert_array_equal(got2, ref2)
    # and the first problem again
    got3, ref3 = _run_both(30000, 256, 602, seed=1)
    np.testing.assert_array_equal(got3, ref)
    np.testing.assert_array_equal(ref3, ref)


def test_noalloc_dw_rejects_sizes_beyond_the_builtin_scratch(cuda):
    from tango_b200 import _lib
    L = _lib.lib
    cap = L.tango_qgemm_dw_noalloc_max_elems()
    assert cap == 1 << 20
    n, k = 2048, 1024                                   # 2 Mi accumulators > capacity
    assert n * k > cap
    rc = L.tango_qgemm_dw_noalloc(None, 2048, None, 1024, 128, n, k, None, None, None, k, None, None)
    assert rc == -5
    assert b"size" in L.tango_strerror(rc)
