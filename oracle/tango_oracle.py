"""CPU restatement (NumPy) of Tango's quantized GNN primitives.

TEST INFRASTRUCTURE ONLY.  This module is the checker the parity tests, the
smoke test and the benchmark's CPU leg compare the CUDA library against; no
product code path may import it.

PARITY UNPINNED: the reference repository ships no golden vectors, known-answer
tests or fixtures for this path, and its kernels are CUDA-only (they cannot run
where this oracle is developed).  Every function below is therefore a
restatement of the arithmetic read off the reference sources, cited per
function as ``file:line`` inside the reference project.  The two input recipes
the reference keeps under ``#ifdef TEST`` (cuda/src/QGEMM_forward.cu:162-181 and
cuda/src/SDDMM.cu:230-257) are reproduced by ``recipe_*`` helpers and used as
committed fixtures.

Arithmetic conventions (what "bit-exact" means for the CUDA side):
  * all fp32 operations are single IEEE-754 round-to-nearest operations with no
    fused multiply-add, in the order written here;
  * ``scale = absmax / 127``; ``inv = 1 / scale`` (0 when scale == 0);
  * integer accumulators are exact (int32 wrap-around is asserted not to occur).
The reference itself is compiled with --use_fast_math (cuda/kernels.py:13), so
its own divisions are approximate; bit-exactness is defined against this file.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
ROUND_TRUNC, ROUND_NEAREST, ROUND_STOCHASTIC = 0, 1, 2

# ----------------------------------------------------------------------------
# Philox4x32-10 counter-based generator (Salmon et al., SC'11) -- public
# algorithm; constants are the published ones.
# ----------------------------------------------------------------------------
_PH_M0 = np.uint64(0xD2511F53)
_PH_M1 = np.uint64(0xCD9E8D57)
_PH_W0 = np.uint32(0x9E3779B9)
_PH_W1 = np.uint32(0xBB67AE85)
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Vectorised Philox4x32-10.  Counters are uint32 arrays (broadcastable),
    keys are uint32 scalars.  Returns four uint32 arrays."""
    c0 = np.asarray(c0, dtype=np.uint32).copy()
    c1 = np.broadcast_to(np.asarray(c1, dtype=np.uint32), c0.shape).copy()
    c2 = np.broadcast_to(np.asarray(c2, dtype=np.uint32), c0.shape).copy()
    c3 = np.broadcast_to(np.asarray(c3, dtype=np.uint32), c0.shape).copy()
    k0 = np.uint32(k0)
    k1 = np.uint32(k1)
    with np.errstate(over="ignore"):
        for _ in range(10):
            p0 = _PH_M0 * c0.astype(np.uint64)
            p1 = _PH_M1 * c2.astype(np.uint64)
            hi0 = (p0 >> np.uint64(32)).astype(np.uint32)
            lo0 = (p0 & _MASK32).astype(np.uint32)
            hi1 = (p1 >> np.uint64(32)).astype(np.uint32)
            lo1 = (p1 & _MASK32).astype(np.uint32)
            n0 = hi1 ^ c1 ^ k0
            n1 = lo1
            n2 = hi0 ^ c3 ^ k1
            n3 = lo0
            c0, c1, c2, c3 = n0, n1, n2, n3
            k0 = np.uint32(k0 + _PH_W0)
            k1 = np.uint32(k1 + _PH_W1)
    return c0, c1, c2, c3


def stochastic_uniforms(numel: int, seed: int, call: int) -> np.ndarray:
    """u in [0,1) for flat element index i: Philox counter = (i//4 lo, i//4 hi,
    call lo, call hi), key = (seed lo, seed hi); lane i%4 of the four outputs;
    u = (r >> 8) * 2^-24."""
    n4 = (numel + 3) // 4
    idx = np.arange(n4, dtype=np.uint64)
    c0 = (idx & _MASK32).astype(np.uint32)
    c1 = (idx >> np.uint64(32)).astype(np.uint32)
    c2 = np.uint32(call & 0xFFFFFFFF)
    c3 = np.uint32((call >> 32) & 0xFFFFFFFF)
    r = philox4x32_10(c0, c1, c2, c3, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    r = np.stack(r, axis=1).reshape(-1)[:numel]
    return (r >> np.uint32(8)).astype(F32) * F32(2.0 ** -24)


# ----------------------------------------------------------------------------
# Quantisation
# ----------------------------------------------------------------------------
def absmax_scale(x: np.ndarray) -> np.float32:
    """scale = max|x| / 127 as one fp32 division.
    Follows cuda/src/quantization.cu:45-93 (kernel_get_scale, get_scale_impl)
    and cuda/src/utils.h:83-99 (scale_reduce); the max is order independent."""
    x = np.asarray(x, dtype=F32)
    m = F32(np.max(np.abs(x))) if x.size else F32(0)
    return F32(m / F32(127.0))


def inv_scale(scale) -> np.float32:
    """1/scale as one fp32 division; 0 when scale is 0 or so small (subnormal) that the reciprocal overflows -- a
    tensor whose absmax is below ~4e-37 quantizes to all zeros instead of producing inf * 0 = NaN."""
    s = F32(scale)
    if s == 0:
        return F32(0)
    with np.errstate(over="ignore"):
        inv = F32(F32(1.0) / s)
    return inv if np.isfinite(inv) else F32(0)


def quantize(x: np.ndarray, scale, mode: int = ROUND_NEAREST, seed: int = 0,
             call: int = 0) -> np.ndarray:
    """int8 = clamp(round_mode(x * (1/scale)), -127, 127).

    nearest: cuda/src/quantization.cu:6-35 (rintf = round half to even, clamp);
    trunc:   cuda/src/iterator.h:155-164 ((int8_t)(x * div_scale), C cast);
    stochastic: not in the reference; floor(x*inv + u) with the Philox stream of
    ``stochastic_uniforms`` indexed by the flat (row-major) element index.
    The off-by-one tail of the reference's nearest kernel
    (cuda/src/quantization.cu:29-34) is not replicated."""
    x = np.asarray(x, dtype=F32)
    inv = inv_scale(scale)
    t = (x * inv).astype(F32)
    if mode == ROUND_NEAREST:
        r = np.rint(t)
    elif mode == ROUND_TRUNC:
        r = np.trunc(t)
    elif mode == ROUND_STOCHASTIC:
        u = stochastic_uniforms(x.size, seed, call).reshape(x.shape)
        r = np.floor((t + u).astype(F32))
    else:
        raise ValueError(mode)
    return np.clip(r, -127, 127).astype(np.int8)


def transpose_quant(e: np.ndarray, scale) -> np.ndarray:
    """fp32 [E,H,D] -> int8 [H,D,E], nearest.  cuda/src/quantization.cu:95-129
    (the reference omits the clamp; values cannot exceed 127 when ``scale`` is
    the tensor's own absmax scale, so the clamp here is a no-op there) and
    cuda/kernels.py:114-119."""
    e = np.asarray(e, dtype=F32)
    assert e.ndim == 3
    q = quantize(e, scale, ROUND_NEAREST)
    return np.ascontiguousarray(np.transpose(q, (1, 2, 0)))


# ----------------------------------------------------------------------------
# int8 GEMMs
# ----------------------------------------------------------------------------
def _igemm(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Exact integer matmul via float64 BLAS (|sum| < 2^53), returned as int64
    after asserting it fits int32 like the device accumulator."""
    acc = a.astype(np.float64) @ b.astype(np.float64)
    assert np.all(np.abs(acc) < 2.0 ** 31), "int32 accumulator would overflow"
    return acc.astype(np.int64)


def qgemm_acc_nt(xq: np.ndarray, wq: np.ndarray) -> np.ndarray:
    """int32 accumulators of X_q[M,K] . W_q[N,K]^T.
    cuda/src/QGEMM_forward.cu:22-27 (A row-major, B column-major = W [N,K])."""
    return _igemm(xq, wq.T)


def dequant(acc: np.ndarray, sa, sb, bias=None) -> np.ndarray:
    """float(acc) * (sa*sb) (+ bias).  cuda/src/epilogue.h:62-100 (Dequant):
    the two scales are multiplied first, then applied; bias is added after."""
    sc = F32(F32(sa) * F32(sb))
    y = (acc.astype(F32) * sc).astype(F32)
    if bias is not None:
        y = (y + np.asarray(bias, dtype=F32)[None, :]).astype(F32)
    return y


def qgemm_forward(x, w, bias=None, mode: int = ROUND_TRUNC, reduce_out: bool = False,
                  seed: int = 0, call: int = 0, sx=None, sw=None):
    """Fused forward of the quantized linear layer.
    cuda/kernels.py:79-94, cuda/src/QGEMM_forward.cu:125-157,
    cuda/src/iterator.h:155-164 (quantize on load, truncating),
    cuda/src/epilogue.h:500-521 (optional output scale = max|Y|/127, bias
    included).  Returns (Y, X_q, W_q, sX, sW, sY or None).  W is [N,K].
    Stochastic mode draws X with call index ``call`` and W with ``call+1``."""
    x = np.asarray(x, dtype=F32)
    w = np.asarray(w, dtype=F32)
    sx = absmax_scale(x) if sx is None else F32(sx)
    sw = absmax_scale(w) if sw is None else F32(sw)
    xq = quantize(x, sx, mode, seed, call)
    wq = quantize(w, sw, mode, seed, call + 1)
    y = dequant(qgemm_acc_nt(xq, wq), sx, sw, bias)
    sy = absmax_scale(y) if reduce_out else None
    return y, xq, wq, sx, sw, sy


def qgemm_backward_dx(dyq, wq, sdy, sw) -> np.ndarray:
    """dX[M,K] = float(dY_q[M,N] . W_q[N,K]) * (s_dY*s_W).
    cuda/src/QGEMM_backward.cu:21-48."""
    return dequant(_igemm(dyq, wq), sdy, sw)


def qgemm_backward_dw(dyq, xq, sdy, sx) -> np.ndarray:
    """dW[N,K] = float(dY_q^T[N,M] . X_q[M,K]) * (s_dY*s_X).
    cuda/src/QGEMM_backward.cu:50-113 (split-K partials are summed in int32
    before the dequantisation, so the split does not change the result)."""
    return dequant(_igemm(dyq.T, xq), sdy, sx)


# ----------------------------------------------------------------------------
# SpMM
# ----------------------------------------------------------------------------
def _shard_of(cols, shard_rows):
    return cols // shard_rows if shard_rows else np.zeros_like(cols)


def spmm_copy_u_acc(indptr, indices, nq) -> np.ndarray:
    """int64 accumulators out[v,:] = sum_{j in row v} N_q[indices[j],:]."""
    n_rows = len(indptr) - 1
    nq2 = nq.reshape(nq.shape[0], -1).astype(np.int64)
    out = np.zeros((n_rows, nq2.shape[1]), dtype=np.int64)
    rows = np.repeat(np.arange(n_rows), np.diff(indptr))
    np.add.at(out, rows, nq2[indices])
    return out


def spmm_copy_u(indptr, indices, nq, scale, shard_rows: int = 0) -> np.ndarray:
    """out[v] = s * sum_{u in row v} N_q[u]  (fp32 [rows, F]).
    cuda/kernels.py:154-165 and cuda/src/SPMM.cu:23-68 (cuSPARSE CSR SpMM with
    all-ones values, alpha = scale).  The library accumulates in fp32; the sum
    of int8 values is exact in either form while it stays below 2^24, so this
    restatement accumulates exactly in integers and scales once.

    ``scale`` may be an array of per-shard scales (row-partitioned training):
    source rows [k*shard_rows, (k+1)*shard_rows) carry scale[k]; per-shard
    integer sums are scaled and then added in increasing shard order in fp32."""
    scale = np.atleast_1d(np.asarray(scale, dtype=F32))
    nq2 = nq.reshape(nq.shape[0], -1)
    if scale.size == 1:
        acc = spmm_copy_u_acc(indptr, indices, nq2)
        assert np.all(np.abs(acc) < 2 ** 31)
        return (acc.astype(F32) * scale[0]).astype(F32)
    n_rows = len(indptr) - 1
    out = np.zeros((n_rows, nq2.shape[1]), dtype=F32)
    rows = np.repeat(np.arange(n_rows), np.diff(indptr))
    sh = _shard_of(np.asarray(indices), shard_rows)
    for k in range(scale.size):
        m = sh == k
        acc = np.zeros((n_rows, nq2.shape[1]), dtype=np.int64)
        np.add.at(acc, rows[m], nq2[indices[m]].astype(np.int64))
        present = np.zeros(n_rows, dtype=bool)
        present[rows[m]] = True
        contrib = (acc.astype(F32) * scale[k]).astype(F32)
        out = np.where(present[:, None], (out + contrib).astype(F32), out)
    return out


def spmm_u_mul_e(indptr, indices, edge_ids, nq, eq, scale) -> np.ndarray:
    """out[v,h,:] = scale * sum_j E_q[eid[j],h] * N_q[indices[j],h,:].
    nq int8 [Nn,H,D]; eq int8 [E,H] in edge-id order; edge_ids maps CSR slot ->
    edge id (None = identity).  cuda/kernels.py:122-136 (index_select by
    edge_ids) and cuda/src/SPMM.cu:70-130 (one cuSPARSE SpMM per head)."""
    n_rows = len(indptr) - 1
    nn, h, d = nq.shape
    if edge_ids is None:
        edge_ids = np.arange(len(indices))
    w = eq.reshape(eq.shape[0], h).astype(np.int64)[edge_ids]          # [nnz,H]
    msg = nq.astype(np.int64)[indices] * w[:, :, None]                 # [nnz,H,D]
    acc = np.zeros((n_rows, h, d), dtype=np.int64)
    rows = np.repeat(np.arange(n_rows), np.diff(indptr))
    np.add.at(acc, rows, msg)
    assert np.all(np.abs(acc) < 2 ** 31)
    return (acc.astype(F32) * F32(scale)).astype(F32)


def spmm_incidence(indptr, edge_ids, zq, scale) -> np.ndarray:
    """out[v,:] = s * sum_{e incident to v} Z_q[e,:]; the incidence structure is
    given as a CSR/CSC (indptr, edge_ids).  cuda/kernels.py:139-152 and
    cuda/src/SPMM.cu:259-303 (COO incidence matrix with all-ones values: row =
    node, column = edge id)."""
    n_rows = len(indptr) - 1
    z2 = zq.reshape(zq.shape[0], -1).astype(np.int64)
    if edge_ids is None:
        edge_ids = np.arange(z2.shape[0])
    acc = np.zeros((n_rows, z2.shape[1]), dtype=np.int64)
    rows = np.repeat(np.arange(n_rows), np.diff(indptr))
    np.add.at(acc, rows, z2[edge_ids])
    return (acc.astype(F32) * F32(scale)).astype(F32)


# ----------------------------------------------------------------------------
# SDDMM
# ----------------------------------------------------------------------------
def sddmm_dot_acc(src, dst, uq, vq) -> np.ndarray:
    """int accumulators [E,H] of sum_d U_q[src,h,d]*V_q[dst,h,d]."""
    return np.einsum("ehd,ehd->eh", uq.astype(np.int64)[src], vq.astype(np.int64)[dst])


def sddmm_dot(src, dst, uq, vq, su, sv) -> np.ndarray:
    """out[e,h] = float(dot) * (sU*sV).  cuda/src/SDDMM.cu:8-47 (int32 dot,
    shuffle reduction, scale = sU*sV applied once)."""
    sc = F32(F32(su) * F32(sv))
    return (sddmm_dot_acc(src, dst, uq, vq).astype(F32) * sc).astype(F32)


def sddmm_elementwise(op: str, src, dst, uq, vq, su, sv) -> np.ndarray:
    """out[e,:] = op(float(U_q[src,:])*sU, float(V_q[dst,:])*sV) in fp32.
    cuda/src/SDDMM.cu:65-100 (kernel_SDDMM_int8)."""
    a = (uq.reshape(uq.shape[0], -1)[src].astype(F32) * F32(su)).astype(F32)
    b = (vq.reshape(vq.shape[0], -1)[dst].astype(F32) * F32(sv)).astype(F32)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = {"add": a + b, "sub": a - b, "mul": a * b, "div": a / b}[op]
    return r.astype(F32)


# ----------------------------------------------------------------------------
# Edge softmax (fp32; not quantised by the reference -- it calls
# dgl.ops.edge_softmax, evaluation/test_gat.py:144-146).  Parity for this op is
# tolerance based (1e-3 relative), not bit-exact: exp is not correctly rounded.
# ----------------------------------------------------------------------------
def leaky_relu(x, slope=0.2):
    x = np.asarray(x, dtype=F32)
    return np.where(x >= 0, x, (x * F32(slope)).astype(F32)).astype(F32)


def edge_softmax(indptr_csc, edge_ids_csc, z) -> np.ndarray:
    """a[e,h] = exp(z[e,h]-max_v)/sum over the incoming edges of dst(e)."""
    z = np.asarray(z, dtype=np.float64)
    out = np.zeros_like(z)
    for v in range(len(indptr_csc) - 1):
        sl = edge_ids_csc[indptr_csc[v]:indptr_csc[v + 1]]
        if len(sl) == 0:
            continue
        zz = z[sl]
        ex = np.exp(zz - zz.max(axis=0, keepdims=True))
        out[sl] = ex / ex.sum(axis=0, keepdims=True)
    return out.astype(F32)


# ----------------------------------------------------------------------------
# Input recipes kept by the reference under #ifdef TEST
# ----------------------------------------------------------------------------
def recipe_gemm_inputs(m: int, n: int, k: int):
    """A[i] = ((i+41)*16807 % 16) - 8, B[i] = ((i+17)*16807 % 16) - 8 as fp32,
    scales 0.5 (cuda/src/QGEMM_forward.cu:162-181,192-210)."""
    ia = np.arange(m * k, dtype=np.int64)
    ib = np.arange(n * k, dtype=np.int64)
    a = (((ia + 41) * 16807) % 16 - 8).astype(F32).reshape(m, k)
    b = (((ib + 17) * 16807) % 16 - 8).astype(F32).reshape(n, k)
    return a, b, F32(0.5), F32(0.5)


def recipe_sddmm_inputs(dim: int, out_len: int = 1):
    """3 nodes, 4 edges (0,0),(0,1),(0,2),(1,2); U[i]=i, V[i]=dim*3*out_len-i as
    int8 (wrapping), scales 1.0 (cuda/src/SDDMM.cu:230-257)."""
    nv = 3
    n = dim * nv * out_len
    u = np.arange(n, dtype=np.int64).astype(np.int8).reshape(nv, out_len, dim)
    v = (n - np.arange(n, dtype=np.int64)).astype(np.int8).reshape(nv, out_len, dim)
    src = np.array([0, 0, 0, 1], dtype=np.int32)
    dst = np.array([0, 1, 2, 2], dtype=np.int32)
    return src, dst, u, v, F32(1.0), F32(1.0)


# ----------------------------------------------------------------------------
# The quantized GCN layer, forward and backward, as a chain of the primitives
# above ("multiply first" branch, norm='both': in_feats > out_feats).
# ----------------------------------------------------------------------------
def gcn_layer_forward(csc, out_norm, in_norm, x, w, b, relu: bool):
    """evaluation/test_gcn.py:86-137: X * d_out^-1/2 -> Qlinear_func_reduce
    (cuda/QLinear.py:50-60: truncating fused forward, output scale) ->
    spmm_copy_u with that scale (cuda/SPMM.py:8-16: nearest quantizer, CSC
    aggregation) -> * d_in^-1/2 -> + bias -> activation.
    csc = (indptr, indices) with rows = destinations.  Returns (out, cache)."""
    xs = (np.asarray(x, F32) * np.asarray(out_norm, F32)[:, None]).astype(F32)
    h, xq, wq, sx, sw, sh = qgemm_forward(xs, w, reduce_out=True)
    hq = quantize(h, sh)
    agg = spmm_copy_u(csc[0], csc[1], hq, sh)
    out = (agg * np.asarray(in_norm, F32)[:, None]).astype(F32)
    if b is not None:
        out = (out + np.asarray(b, F32)[None, :]).astype(F32)
    if relu:
        out = np.maximum(out, F32(0))
    return out, dict(xq=xq, wq=wq, sx=sx, sw=sw, out=out, relu=relu, has_bias=b is not None)


def gcn_layer_backward(csr, out_norm, in_norm, cache, d_out, need_dx: bool = True):
    """Backward of gcn_layer_forward, operator by operator as autograd runs the
    reference's layer: ReLU mask; bias gradient = column sums in fp32; right
    norm; spmm_copy_u.backward (cuda/SPMM.py:18-24: nearest quantizer with the
    gradient's own scale, aggregation over the CSR = reversed graph);
    Qlinear_func_reduce.backward (cuda/QLinear.py:62-72: dY_q nearest, dX and dW
    from the cached int8 operands); left norm.  csr = (indptr, indices) with
    rows = sources.  Returns (dX or None, dW, db or None)."""
    g = np.asarray(d_out, F32)
    if cache["relu"]:
        g = np.where(cache["out"] > 0, g, F32(0)).astype(F32)
    db = g.astype(np.float64).sum(0).astype(F32) if cache["has_bias"] else None
    gz = (g * np.asarray(in_norm, F32)[:, None]).astype(F32)
    sdz = absmax_scale(gz)
    dh = spmm_copy_u(csr[0], csr[1], quantize(gz, sdz), sdz)
    sdh = absmax_scale(dh)
    dhq = quantize(dh, sdh)
    dw = qgemm_backward_dw(dhq, cache["xq"], sdh, cache["sx"])
    dx = None
    if need_dx:
        dx = (qgemm_backward_dx(dhq, cache["wq"], sdh, cache["sw"]) * np.asarray(out_norm, F32)[:, None]).astype(F32)
    return dx, dw, db


def cross_entropy_mean(logits, labels):
    """Mean cross-entropy over all rows and its gradient with respect to the
    logits (float64 internally; torch.nn.functional.cross_entropy as used at
    evaluation/test_gcn.py:257, without the train mask synthetic data lacks)."""
    z = np.asarray(logits, np.float64)
    z = z - z.max(axis=1, keepdims=True)
    lse = np.log(np.exp(z).sum(axis=1, keepdims=True))
    logp = z - lse
    n = z.shape[0]
    loss = -logp[np.arange(n), labels].mean()
    grad = np.exp(logp)
    grad[np.arange(n), labels] -= 1.0
    return F32(loss), (grad / n).astype(F32)
