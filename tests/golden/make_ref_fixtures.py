"""Produces tests/golden/ref_fixtures.npz: outputs of the REFERENCE's own CUDA kernels on seeded inputs.

Runs on a machine with a CUDA device and the module built by oracle/build_ref.py (the reference's
cuda/src/quantization.cu, SDDMM.cu, QGEMM_backward.cu and SPMM.cu compiled with its own flags):

    python tests/golden/make_ref_fixtures.py OUT.npz

The file holds inputs and outputs; tests/test_oracle.py checks the CPU oracle against it, which is what pins the
oracle to the reference.  Inputs respect what the reference's kernels can take: every fp32 tensor has a multiple of
four elements (its tail path reads one element past the buffer, cuda/src/quantization.cu:29-34), GEMM leading
dimensions are multiples of four, indices are int64.  The cuSPARSE calls run in a child process so that a library
status the reference answers with exit() cannot lose the other fixtures; its COO incidence call is not run at all
(it hands cuSPARSE a null workspace, cuda/src/SPMM.cu:296-298).
"""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def _graph(rng, n, e):
    src = rng.integers(0, n, e).astype(np.int64)
    dst = rng.integers(0, n, e).astype(np.int64)
    return src, dst


def main_kernels(out_path):
    import torch
    from oracle import build_ref
    ref = build_ref.load()
    assert ref is not None, "build oracle/_ref first (python oracle/build_ref.py)"
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(20241125)
    fx = {}

    def T(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    # ---- get_scale / quantize (nearest), natural scale and a power-of-two scale (exact reciprocal under fast-math)
    x = rng.standard_normal((96, 64)).astype(np.float32) * 3.0
    xt = T(x)
    s = ref.get_scale(xt)
    q = torch.empty(x.shape, dtype=torch.int8, device=dev)
    ref.quantize(q, xt, s)
    fx["q_x"], fx["q_scale"], fx["q_out"] = x, s.cpu().numpy(), q.cpu().numpy()
    s2 = T(np.array([0.0625], dtype=np.float32))
    q2 = torch.empty(x.shape, dtype=torch.int8, device=dev)
    ref.quantize(q2, xt, s2)
    fx["q_out_pow2"] = q2.cpu().numpy()
    half = (rng.integers(-200, 200, (32, 16)).astype(np.float32) + 0.5) * 0.0625     # exact .5 ties after scaling
    q3 = torch.empty(half.shape, dtype=torch.int8, device=dev)
    ref.quantize(q3, T(half), s2)
    fx["q_ties_x"], fx["q_ties_out"] = half, q3.cpu().numpy()
    # ---- transpose_quant: [E, H, D] -> [H*D, E]
    for tag, shape in (("a", (300, 4, 1)), ("b", (52, 2, 8))):
        e = rng.random(shape).astype(np.float32)
        et = T(e)
        se = ref.get_scale(et)
        out = ref.transpose_quant(et, se, shape[0], shape[1] * shape[2])
        fx[f"tq_{tag}_x"], fx[f"tq_{tag}_scale"], fx[f"tq_{tag}_out"] = e, se.cpu().numpy(), out.cpu().numpy()
    # ---- SDDMM dot and element-wise
    n, ne = 200, 1500
    src, dst = _graph(rng, n, ne)
    fx["sd_src"], fx["sd_dst"] = src, dst
    st, dt = T(src), T(dst)
    for tag, (h, d) in (("h4d16", (4, 16)), ("h1d70", (1, 70)), ("h2d33", (2, 33))):
        u = rng.integers(-127, 128, (n, h, d)).astype(np.int8)
        v = rng.integers(-127, 128, (n, h, d)).astype(np.int8)
        su, sv = np.array([0.013], dtype=np.float32), np.array([0.021], dtype=np.float32)
        out = torch.empty((ne, h, 1), dtype=torch.float32, device=dev)
        so = torch.zeros(1, dtype=torch.float32, device=dev)
        ref.mySDDMM_int8("dot", out, so, st, dt, T(u), T(v), T(su), T(sv))
        fx[f"sd_{tag}_u"], fx[f"sd_{tag}_v"], fx[f"sd_{tag}_su"], fx[f"sd_{tag}_sv"] = u, v, su, sv
        fx[f"sd_{tag}_out"], fx[f"sd_{tag}_scale_out"] = out.cpu().numpy(), so.cpu().numpy()
    u = rng.integers(-127, 128, (n, 4, 1)).astype(np.int8)
    v = rng.integers(1, 128, (n, 4, 1)).astype(np.int8)          # positive: 'div' stays finite
    su, sv = np.array([0.03], dtype=np.float32), np.array([0.017], dtype=np.float32)
    fx["se_u"], fx["se_v"], fx["se_su"], fx["se_sv"] = u, v, su, sv
    for op in ("add", "sub", "mul", "div"):
        out = torch.empty((ne, 4, 1), dtype=torch.float32, device=dev)
        ref.mySDDMM_int8(op, out, torch.empty(0, device=dev), st, dt, T(u), T(v), T(su), T(sv))
        fx[f"se_{op}_out"] = out.cpu().numpy()
    # ---- backward GEMMs (CUTLASS SIMT int8): dX = dY . W, dW = dY^T . X (split-K when M > 4 N)
    for tag, (m, nn, k) in (("a", (512, 64, 128)), ("b", (96, 64, 100))):
        dy = rng.integers(-127, 128, (m, nn)).astype(np.int8)
        w = rng.integers(-127, 128, (nn, k)).astype(np.int8)
        xq = rng.integers(-127, 128, (m, k)).astype(np.int8)
        sdy, sw, sx = (np.array([v_], dtype=np.float32) for v_ in (0.011, 0.0023, 0.037))
        dx = torch.empty((m, k), dtype=torch.float32, device=dev)
        ref.QGEMM_backward_gradX(dx, T(dy), T(w), T(sdy), T(sw))
        dw = torch.empty((nn, k), dtype=torch.float32, device=dev)
        ref.QGEMM_backward_gradW(dw, T(dy), T(xq), T(sdy), T(sx))
        for name, val in (("dy", dy), ("w", w), ("x", xq), ("sdy", sdy), ("sw", sw), ("sx", sx),
                          ("dx", dx.cpu().numpy()), ("dw", dw.cpu().numpy())):
            fx[f"bg_{tag}_{name}"] = val
    torch.cuda.synchronize()
    np.savez_compressed(out_path, **fx)
    print("kernels:", len(fx), "arrays ->", out_path)


def main_cusparse(out_path):
    """csr_SPMM and multi_cusparse_SPMM of the reference (cuSPARSE, int8 operands, fp32 compute)."""
    import torch
    from oracle import build_ref
    ref = build_ref.load()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(77)
    fx = {}

    def T(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    n, ne = 300, 4000
    src, dst = _graph(rng, n, ne)
    order = np.lexsort((src, dst))               # CSC: rows = destinations, columns = sources
    src, dst = src[order], dst[order]
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(dst, minlength=n), out=indptr[1:])
    fx["sp_indptr"], fx["sp_indices"] = indptr, src
    nq = rng.integers(-127, 128, (n, 64)).astype(np.int8)
    sc = np.array([0.019], dtype=np.float32)
    out = torch.zeros((n, 64), dtype=torch.float32, device=dev)
    ref.csr_SPMM(out, T(indptr), T(src), T(nq), T(sc))
    fx["sp_nq"], fx["sp_scale"], fx["sp_copy_u_out"] = nq, sc, out.cpu().numpy()
    n3 = rng.integers(-127, 128, (n, 4, 16)).astype(np.int8)
    e_t = rng.integers(-127, 128, (4, 1, ne)).astype(np.int8)    # already in CSC-slot order
    out3 = ref.multi_cusparse_SPMM(T(indptr), T(src), T(n3), T(e_t), T(sc))
    fx["sp_n3"], fx["sp_e_t"], fx["sp_u_mul_e_out"] = n3, e_t, out3.cpu().numpy()
    torch.cuda.synchronize()
    np.savez_compressed(out_path, **fx)
    print("cusparse:", len(fx), "arrays ->", out_path)


if __name__ == "__main__":
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_fixtures.npz")
    if len(sys.argv) > 2 and sys.argv[2] == "--cusparse-child":
        main_cusparse(out)
        sys.exit(0)
    main_kernels(out)
    side = out.replace(".npz", "_cusparse.npz")
    rc = subprocess.run([sys.executable, os.path.abspath(__file__), side, "--cusparse-child"], timeout=600).returncode
    print("cusparse child exit code", rc)
