"""Python wrappers with the names and signatures of the reference's cuda/kernels.py, backed by the prebuilt
sm_100a library instead of a runtime JIT of CUTLASS sources (cuda/kernels.py:10-16 in the reference).

`cuda_kernels` mirrors the reference's pybind module (cuda/src/cuda.cpp:182-204): scripts call
`cuda_kernels.get_scale(t)` directly.  The free functions below mirror cuda/kernels.py:19-178.

Differences a caller can observe:
  * graph index tensors are int32;
  * int8 tensors whose row width is not a multiple of 16 bytes are returned as views of zero-padded storage
    (same shape, row stride rounded up to 16) so that every kernel can use 128-bit accesses and TMA;
  * `quantize`/`QGEMM_forward` accept `mode`/`seed`/`call` for the rounding mode (defaults reproduce the
    reference: nearest for `quantize`, truncation for the fused forward).
"""
from __future__ import annotations

import ctypes
import types
from typing import Optional

import torch

from . import _lib, config
from ._lib import ROUND_NEAREST, ROUND_STOCHASTIC, ROUND_TRUNC, SpmmPlan, check, lib
from .graph import SpmmSchedule

__all__ = ["cuda_kernels", "quantize", "mySDDMM_int8", "QGEMM_forward", "QGEMM_backward", "transpose_quant",
           "multi_cusparse_SPMM", "incidence_SPMM", "csr_SPMM", "multi_cusparse_SPMV", "infer_broadcast_shape",
           "ROUND_TRUNC", "ROUND_NEAREST", "ROUND_STOCHASTIC", "device_status", "alloc_int8"]


# --------------------------------------------------------------------------------------------------- plumbing
def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t: Optional[torch.Tensor]):
    return None if t is None or t.numel() == 0 else t.data_ptr()


_dummy_index = {}      # device -> one int32 zero, the address handed over for empty index arrays


def _pi(t: torch.Tensor):
    """Pointer of a mandatory index array; an empty one (graph without edges) still needs a valid address."""
    if t.numel() == 0:
        d = _dummy_index.get(t.device)
        if d is None:
            d = _dummy_index[t.device] = torch.zeros(1, dtype=torch.int32, device=t.device)
        return d.data_ptr()
    return t.data_ptr()


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def _matrix(t: torch.Tensor):
    """(tensor, rows, cols, ld): `t` seen as a row-major [rows, cols] matrix with leading dimension ld (elements)."""
    rows = t.shape[0] if t.dim() else 1
    cols = t.numel() // rows if rows else 0
    if t.dim() <= 1:
        t = t.contiguous()
        return t, 1, t.numel(), max(t.numel(), 1)
    if t.is_contiguous():
        return t, rows, cols, max(cols, 1)
    if rows > 0 and t[0].is_contiguous() and t.stride(0) >= cols:
        return t, rows, cols, t.stride(0)
    t = t.contiguous()
    return t, rows, cols, max(cols, 1)


def alloc_int8(shape, device, align: int = 16) -> torch.Tensor:
    """int8 tensor of `shape` whose rows (dim 0) are padded to a multiple of `align` bytes: 16 for GEMM operands and
    gathered feature rows (TMA and 128-bit loads), 4 is enough for per-head edge or node scalars."""
    shape = tuple(shape)
    if len(shape) < 2:
        return torch.empty(shape, dtype=torch.int8, device=device)
    rows, cols = shape[0], 1
    for s in shape[1:]:
        cols *= s
    ld = _round_up(max(cols, 1), align)
    store = torch.empty((rows, ld), dtype=torch.int8, device=device)
    if ld == cols:
        return store.view(shape)
    v = store[:, :cols]
    return v.unflatten(1, shape[1:]) if len(shape) > 2 else v


_status = {}


def device_status(device=None, reset: bool = False) -> int:
    """Value of the per-device status word written by kernels with bounded waits (0 = no timeout).  Synchronises."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    t = _status.get(dev)
    if t is None:
        return 0
    v = int(t.item())
    if reset:
        t.zero_()
    return v


def _status_word(device) -> torch.Tensor:
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    t = _status.get(dev)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[dev] = t
    return t


launch_counter = [0]  # kernels of this library launched so far (benchmarks report it per step)
_call_counter = [0]


def next_call() -> int:
    """Monotonic per-process counter that keys the stochastic-rounding stream of successive calls."""
    _call_counter[0] += 1
    return _call_counter[0]


def set_call_counter(v: int) -> None:
    _call_counter[0] = int(v)


def infer_broadcast_shape(op, ushape, vshape):
    """Trailing-shape broadcast used by the SDDMM wrapper (dgl.sparse.infer_broadcast_shape in the reference,
    cuda/kernels.py:3,49-50): NumPy broadcast, with the last dimension collapsed to 1 for 'dot'."""
    ushape, vshape = tuple(ushape), tuple(vshape)
    if op == "dot" and ushape[-1] != vshape[-1]:
        raise ValueError("dot needs equal feature sizes")
    n = max(len(ushape), len(vshape))
    u = (1,) * (n - len(ushape)) + ushape
    v = (1,) * (n - len(vshape)) + vshape
    out = []
    for a, b in zip(u, v):
        if a != b and a != 1 and b != 1:
            raise ValueError(f"cannot broadcast {ushape} with {vshape}")
        out.append(max(a, b))
    if op == "dot":
        out[-1] = 1
    return tuple(out)


# --------------------------------------------------------------------------------------------------- native module
def _get_scale(t: torch.Tensor, row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert t.is_cuda and t.dtype == torch.float32
    t, rows, cols, ld = _matrix(t)
    scale = torch.empty(1, dtype=torch.float32, device=t.device)
    with torch.cuda.device(t.device):
        check(lib.tango_absmax_scale(_p(t), rows, cols, ld, _p(row_scale), _p(scale), _stream()), "get_scale")
    launch_counter[0] += 1
    return scale


def _quantize_into(out: torch.Tensor, t: torch.Tensor, scale: torch.Tensor, mode: int = ROUND_NEAREST, seed: int = 0,
                   call: int = 0, row_scale: Optional[torch.Tensor] = None) -> None:
    assert t.is_cuda and out.is_cuda and out.dtype == torch.int8 and t.dtype == torch.float32
    assert out.shape == t.shape
    t, rows, cols, ldx = _matrix(t)
    o2, orows, ocols, ldq = _matrix(out)
    assert o2.data_ptr() == out.data_ptr(), "output int8 tensor must be row-strided, not arbitrary-strided"
    with torch.cuda.device(t.device):
        check(lib.tango_quantize(_p(t), rows, cols, ldx, _p(row_scale), _p(scale), _p(out), ldq, mode, seed, call,
                                 _p(config.step_counter()), _stream()), "quantize")
    launch_counter[0] += 1


def _transpose_quant(data: torch.Tensor, scale: torch.Tensor, nrow: int, ncol: int) -> torch.Tensor:
    data = data.contiguous()
    out = torch.empty((ncol, nrow), dtype=torch.int8, device=data.device)
    with torch.cuda.device(data.device):
        check(lib.tango_quantize_transpose(_p(data), nrow, ncol, _p(scale), _p(out), _stream()), "transpose_quant")
    launch_counter[0] += 1
    return out


def _qgemm_forward(Y, X, X_q, W, W_q, bias, scaleY, scaleX, scaleW, mode=ROUND_TRUNC, seed=0, call=0, row_scale=None):
    X, m, k, ldx = _matrix(X)
    W, n, k2, ldw = _matrix(W)
    assert k == k2
    _, _, _, ldxq = _matrix(X_q)
    _, _, _, ldwq = _matrix(W_q)
    _, _, _, ldy = _matrix(Y)
    st = _status_word(X.device)
    with torch.cuda.device(X.device):
        check(lib.tango_qgemm_forward(_p(X), ldx, _p(row_scale), _p(W), ldw, m, n, k, _p(scaleX), _p(scaleW), _p(X_q), ldxq, _p(W_q),
                                      ldwq, _p(bias), _p(Y), ldy, _p(scaleY), mode, seed, call, _p(config.step_counter()),
                                      _p(st), _stream()),
              "QGEMM_forward")
    launch_counter[0] += 3


def _qgemm_nt(Y, X_q, W_q, scaleX, scaleW, bias=None, scaleY=None):
    _, m, k, ldx = _matrix(X_q)
    _, n, _, ldw = _matrix(W_q)
    _, _, _, ldy = _matrix(Y)
    st = _status_word(X_q.device)
    with torch.cuda.device(X_q.device):
        check(lib.tango_qgemm_nt(_p(X_q), ldx, _p(W_q), ldw, m, n, k, _p(scaleX), _p(scaleW), _p(bias), _p(Y), ldy,
                                 _p(scaleY), _p(st), _stream()), "qgemm_nt")
    launch_counter[0] += 1


def _qgemm_gradX(dX, dY_q, W_q, scaledY, scaleW, row_scale=None):
    _, m, n, lddy = _matrix(dY_q)
    _, n2, k, ldw = _matrix(W_q)
    assert n == n2
    _, _, _, lddx = _matrix(dX)
    st = _status_word(dX.device)
    with torch.cuda.device(dX.device):
        check(lib.tango_qgemm_dx(_p(dY_q), lddy, _p(W_q), ldw, m, n, k, _p(scaledY), _p(scaleW), _p(row_scale), _p(dX), lddx, _p(st),
                                 _stream()), "QGEMM_backward_gradX")
    launch_counter[0] += 1


def _qgemm_gradW(dW, dY_q, X_q, scaledY, scaleX):
    _, m, n, lddy = _matrix(dY_q)
    _, m2, k, ldx = _matrix(X_q)
    assert m == m2
    _, _, _, lddw = _matrix(dW)
    nbytes = lib.tango_qgemm_dw_workspace_bytes(n, k)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dW.device)
    st = _status_word(dW.device)
    with torch.cuda.device(dW.device):
        check(lib.tango_qgemm_dw(_p(dY_q), lddy, _p(X_q), ldx, m, n, k, _p(scaledY), _p(scaleX), _p(dW), lddw, _p(ws),
                                 nbytes, _p(st), _stream()), "QGEMM_backward_gradW")
    launch_counter[0] += 2


def _make_plan(sched: Optional[SpmmSchedule], f: int, device):
    """ctypes plan + the tensors that must stay alive for the call."""
    if sched is None:
        return None, ()
    order = getattr(sched, "row_order", None)
    order_ptr = order.data_ptr() if order is not None and order.numel() else None
    n_long = getattr(sched, "n_long", -1) if order_ptr else -1
    hub = getattr(sched, "hub", None)
    if sched.n_heavy == 0:
        plan = SpmmPlan(None, 0, None, 0, None, 0, sched.threshold, order_ptr, n_long)
        return ctypes.byref(plan), (plan,)
    ws_ld = _round_up(f, 16)
    ws = torch.empty((sched.n_heavy * sched.nseg, ws_ld), dtype=torch.int32, device=device)
    plan = SpmmPlan(sched.units.data_ptr() if sched.n_units else None, sched.n_units, sched.heavy_rows.data_ptr(),
                    sched.n_heavy, ws.data_ptr(), ws_ld, sched.threshold, order_ptr, n_long)
    keep = [plan, ws]
    if hub is not None:
        packed = torch.empty((hub.cols.numel(), ws_ld), dtype=torch.int8, device=device)
        plan.dense_a, plan.dense_n_tiles, plan.dense_rows = hub.dense.data_ptr(), hub.n_tiles, hub.rows.numel()
        plan.dense_units, plan.dense_n_units = hub.units.data_ptr(), hub.units.shape[0]
        plan.dense_cols, plan.dense_n_cols = hub.cols.data_ptr(), hub.cols.numel()
        plan.dense_b, plan.dense_status = packed.data_ptr(), _status_word(device).data_ptr()
        plan.n_skip_rows = sched.n_skip
        keep.append(packed)
    return ctypes.byref(plan), tuple(keep)


def _csr_spmm(out, indptr, indices, U, scaleU, sched=None, nseg=1, row_scale=None, bias=None, relu=False,
              out_absmax=None):
    U, _, f, ldn = _matrix(U)
    n_rows = (indptr.numel() - 1) // nseg
    _, _, _, ldo = _matrix(out)
    plan, keep = _make_plan(sched, f, U.device)
    with torch.cuda.device(U.device):
        check(lib.tango_spmm_copy_u(_p(indptr), _pi(indices), n_rows, nseg, _p(U), ldn, f, _p(scaleU), _p(row_scale),
                                    _p(bias), int(relu), _p(out), ldo, _p(out_absmax), plan, _stream()), "csr_SPMM")
    launch_counter[0] += (1 + (sched is not None and sched.n_heavy > 0)
                          + (sched is not None and sched.n_long < sched.row_order.numel())
                          + (2 if getattr(sched, "hub", None) is not None else 0))
    del keep


def hub_self_check(hub, indptr, indices, plain_sched, n_feature_rows: int, f: int = 64) -> bool:
    """Aggregates one random int8 table twice -- every edge gathered, and with the dense hub region `hub` on the tensor
    cores -- and says whether the two results are the same bits (they must be: both are exact int32 sums, and with a
    scale of 1 the fp32 outputs are those integers).  Run once when a hub region is built, so that a region that does
    not reproduce the plain aggregation on this graph, device or driver is dropped instead of used."""
    dev = indptr.device
    gen = torch.Generator(device=dev).manual_seed(1234)
    q = torch.randint(-127, 128, (n_feature_rows, f), dtype=torch.int8, device=dev, generator=gen)
    one = torch.ones(1, dtype=torch.float32, device=dev)
    n_rows = indptr.numel() - 1
    ref = torch.empty((n_rows, f), dtype=torch.float32, device=dev)
    got = torch.full((n_rows, f), float("nan"), dtype=torch.float32, device=dev)
    launches, status = launch_counter[0], device_status(dev)
    try:
        _csr_spmm(ref, indptr, indices, q, one, plain_sched, 1)
        _csr_spmm(got, hub.indptr, hub.indices, q, one, hub.schedule, 1)
        ok = bool(torch.equal(ref, got)) and device_status(dev) == status     # no bounded wait of the GEMM expired
    except _lib.TangoError:
        ok = False
    launch_counter[0] = launches
    return ok


def _u_mul_e_spmm(indptr, indices, edge_ids, N, E, scale, sched=None):
    """N int8 [Nn, H, D]; E int8 [nnz or E, H] (edge-id order when edge_ids is given, CSR-slot order otherwise)."""
    assert N.dim() == 3
    nn, h, d = N.shape
    N, _, f, ldn = _matrix(N)
    E = E.contiguous() if E.numel() else torch.zeros(1, dtype=torch.int8, device=N.device)
    n_rows = indptr.numel() - 1
    out = torch.empty((n_rows, h, d), dtype=torch.float32, device=N.device)
    plan, keep = _make_plan(sched, f, N.device)
    with torch.cuda.device(N.device):
        check(lib.tango_spmm_u_mul_e(_p(indptr), _pi(indices), _p(edge_ids), n_rows, _p(N), ldn, h, d, _p(E), _p(scale),
                                     _p(out), f, plan, _stream()), "multi_cusparse_SPMM")
    launch_counter[0] += 1 + (sched is not None and sched.n_units > 0) + (sched is not None and sched.n_long < sched.row_order.numel())
    del keep
    return out


def _incidence_spmm(out, indptr, edge_ids, E, scale, sched=None):
    E, _, f, ldz = _matrix(E)
    n_rows = indptr.numel() - 1
    _, _, _, ldo = _matrix(out)
    plan, keep = _make_plan(sched, f, E.device)
    with torch.cuda.device(E.device):
        check(lib.tango_spmm_incidence(_p(indptr), _p(edge_ids), n_rows, _p(E), ldz, f, _p(scale), _p(out), ldo, plan,
                                       _stream()), "incidence_SPMM")
    contiguous = edge_ids is None and ldz == f and f in (1, 2, 4, 8, 16)    # streamed by the contiguous-row kernel
    has_short = sched is not None and sched.n_long < sched.row_order.numel() and (not contiguous or f in (4, 8, 16))
    launch_counter[0] += 1 + (sched is not None and sched.n_units > 0) + has_short
    del keep


# Average edges per row from which mySDDMM_int8("dot") walks rows.  On a graph with a handful of edges per row the
# endpoint-list kernel (32 edges per warp, whatever their rows) measured faster than the row walk even with its
# lane-group kernel for short rows (169,343 nodes / 1.3 M edges, 4 heads x 32: 0.060 ms against 0.069 ms).
ROWWISE_SDDMM_MIN_DEGREE = 32


def _sddmm_dot_rows(out, scaleOut, indptr, indices, edge_ids, U, V, scaleU, scaleV, sched=None) -> bool:
    """Row-wise dot SDDMM over a CSR/CSC bundle; False when the operand layout needs the endpoint-list kernel."""
    h, d = U.shape[-2], U.shape[-1]
    U2, _, _, ldu = _matrix(U)
    V2, _, _, ldv = _matrix(V)
    n_rows = indptr.numel() - 1
    plan, keep = (None, ())
    if sched is not None:
        order = sched.row_order
        plan_obj = SpmmPlan(sched.units.data_ptr() if sched.n_units else None, sched.n_units, None, 0, None, 0,
                            sched.threshold, order.data_ptr() if order.numel() else None,
                            sched.n_long if order.numel() else -1)
        plan, keep = ctypes.byref(plan_obj), (plan_obj,)
    with torch.cuda.device(U.device):
        rc = lib.tango_sddmm_dot_rows(_p(indptr), _pi(indices), _p(edge_ids), n_rows, _p(U2), ldu, _p(V2), ldv, h, d,
                                      _p(scaleU), _p(scaleV), _p(out), _p(scaleOut), plan, _stream())
    del keep
    if rc == _lib.TANGO_EALIGN:
        return False
    check(rc, "mySDDMM_int8(dot, rows)")
    launch_counter[0] += 1 + (sched is not None and sched.n_long < n_rows)
    return True


def _sddmm(op: str, out, scaleOut, src, dst, U, V, scaleU, scaleV):
    n_edges = src.numel()
    launch_counter[0] += 1
    with torch.cuda.device(U.device):
        if op == "dot":
            h, d = U.shape[-2], U.shape[-1]
            U2, _, _, ldu = _matrix(U)
            V2, _, _, ldv = _matrix(V)
            check(lib.tango_sddmm_dot(_p(src), _p(dst), n_edges, _p(U2), ldu, _p(V2), ldv, h, d, _p(scaleU),
                                      _p(scaleV), _p(out), _p(scaleOut), _stream()), "mySDDMM_int8(dot)")
        elif op in _lib.OPS:
            U2, _, dim, ldu = _matrix(U)
            V2, _, dimv, ldv = _matrix(V)
            assert dim == dimv, "element-wise SDDMM needs equal feature shapes"
            check(lib.tango_sddmm_elementwise(_lib.OPS[op], _p(src), _p(dst), n_edges, _p(U2), ldu, _p(V2), ldv, dim,
                                              _p(scaleU), _p(scaleV), _p(out), _p(scaleOut), _stream()),
                  f"mySDDMM_int8({op})")
        else:
            raise ValueError(f"{op} op not supported")


def _qgemm_generic(kind: str, A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """QgemmNT/NN/TN of the reference's legacy cuBLAS path (cuda/src/Qgemm_impl.cu:107-125): quantise both fp32
    operands (nearest) and multiply.  Thin aliases of the tcgen05 GEMMs, kept for API completeness."""
    sa, sb = _get_scale(A), _get_scale(B)
    Aq, Bq = alloc_int8(A.shape, A.device), alloc_int8(B.shape, B.device)
    _quantize_into(Aq, A, sa)
    _quantize_into(Bq, B, sb)
    if kind == "NT":      # A[M,K] . B[N,K]^T
        out = torch.empty((A.shape[0], B.shape[0]), dtype=torch.float32, device=A.device)
        _qgemm_nt(out, Aq, Bq, sa, sb)
    elif kind == "NN":    # A[M,N] . B[N,K]
        out = torch.empty((A.shape[0], B.shape[1]), dtype=torch.float32, device=A.device)
        _qgemm_gradX(out, Aq, Bq, sa, sb)
    else:                 # A[M,N]^T . B[M,K]
        out = torch.empty((A.shape[1], B.shape[1]), dtype=torch.float32, device=A.device)
        _qgemm_gradW(out, Aq, Bq, sa, sb)
    return out


def _spmv_stub(*args, **kwargs):
    raise NotImplementedError("multi_cusparse_SPMV is an unfinished stub in the reference (cuda/src/SPMM.cu:196-257)")


cuda_kernels = types.SimpleNamespace(
    QGEMM_forward=_qgemm_forward,
    quantize=lambda out, t, scale: _quantize_into(out, t, scale),
    get_scale=_get_scale,
    transpose_quant=_transpose_quant,
    QgemmNT=lambda A, B: _qgemm_generic("NT", A, B),
    QgemmTN=lambda A, B: _qgemm_generic("TN", A, B),
    QgemmNN=lambda A, B: _qgemm_generic("NN", A, B),
    QGEMM_backward_gradX=_qgemm_gradX,
    QGEMM_backward_gradW=_qgemm_gradW,
    csr_SPMM=lambda out, indptr, indices, U, scaleU: _csr_spmm(out, indptr, indices, U, scaleU),
    multi_cusparse_SPMM=lambda indptr, indices, N, E_T, scale: _u_mul_e_spmm(
        indptr, indices, None, N, E_T.reshape(E_T.shape[0], -1).t().contiguous(), scale),
    incidence_SPMM=lambda out, src, dst, E, scale: _incidence_from_coo(out, src, dst, E, scale),
    multi_cusparse_SPMV=_spmv_stub,
    mySDDMM_int8=_sddmm,
)


def _incidence_from_coo(out, nodes, edge_ids, E, scale):
    """Reference signature (cuda/src/SPMM.cu:259-303): COO rows = node ids (sorted, coalesced), cols = edge ids."""
    n = out.shape[0]
    counts = torch.bincount(nodes.long(), minlength=n)
    indptr = torch.zeros(n + 1, dtype=torch.int64, device=nodes.device)
    torch.cumsum(counts, 0, out=indptr[1:])
    _incidence_spmm(out, indptr.to(torch.int32), edge_ids.to(torch.int32).contiguous(), E, scale)


# --------------------------------------------------------------------------------------------------- wrappers
def _bundle(g, reverse: bool):
    """(indptr, indices, edge_ids) of the CSR (reverse) or CSC; edge_ids is None when slot k stores edge k, so the
    kernels skip the indirection (and the 4 bytes per edge it would stream)."""
    indptr, indices, edge_ids = g.adj_csr if reverse else g.adj_csc
    ident = getattr(g, "_identity", None)
    if ident is not None and ident.get("csr" if reverse else "csc", False):
        edge_ids = None
    return indptr, indices, edge_ids


def _schedule(g, reverse: bool) -> Optional[SpmmSchedule]:
    plans = getattr(g, "_plans", None)
    if plans is None:
        return None
    key = "csr" if reverse else "csc"
    if key not in plans:
        indptr = (g.adj_csr if reverse else g.adj_csc)[0]
        plans[key] = SpmmSchedule(indptr)
    return plans[key]


def quantize(t: torch.Tensor, scale: torch.Tensor = None, mode: int = ROUND_NEAREST, seed: int = 0,
             call: Optional[int] = None, align: int = 16):
    """Quantize the input tensor to 8-bit (cuda/kernels.py:19-30).  Returns (int8 tensor, scale)."""
    assert t.is_cuda, "tensor must be on GPU"
    if scale is None:
        scale = cuda_kernels.get_scale(t)
    out = alloc_int8(t.shape, t.device, align)
    if mode == ROUND_STOCHASTIC and call is None:
        call = next_call()
    _quantize_into(out, t, scale, mode, seed, call or 0)
    return out, scale


def mySDDMM_int8(g, op, U, V, scaleU, scaleV, isReduce, reverse=False):
    """cuda/kernels.py:33-59."""
    if reverse:
        dst, src = g.coo
    else:
        src, dst = g.coo
    assert src.is_cuda and dst.is_cuda and U.is_cuda and V.is_cuda and scaleU.is_cuda and scaleV.is_cuda
    UV_unsqueezed = False
    if len(U.shape) == 2 and len(V.shape) == 2:
        U = U.unsqueeze(1)
        V = V.unsqueeze(1)
        UV_unsqueezed = True
    out_shape = (src.size(0),) + infer_broadcast_shape(op, U.shape[1:], V.shape[1:])
    out = torch.empty(out_shape, dtype=torch.float32, device=src.device)
    scale = torch.zeros((1,), dtype=torch.float32, device=src.device) if isReduce else torch.Tensor()
    done = False
    if (op == "dot" and src.numel() > 0 and src.numel() >= ROWWISE_SDDMM_MIN_DEGREE * g.num_nodes() and U.shape[1:] == V.shape[1:]
            and U.dim() == 3 and U.shape[0] == g.num_nodes() == V.shape[0]):
        # walk the rows of the fixed endpoint: V's row stays in registers, only U is gathered (half the gathered
        # bytes of the endpoint-list kernel, and half its index stream); long rows get a warp, the few short rows of
        # such a graph a group of lanes each.
        indptr, indices, edge_ids = _bundle(g, reverse)
        done = _sddmm_dot_rows(out, scale, indptr, indices, edge_ids, U, V, scaleU, scaleV, _schedule(g, reverse))
    if not done:
        cuda_kernels.mySDDMM_int8(op, out, scale, src, dst, U, V, scaleU, scaleV)
    if UV_unsqueezed:
        out = out.squeeze(1)
    return out, scale


def QGEMM_forward(x, x_, scaleX, w, w_, scaleW, bias=None, isReduce=False, mode: int = ROUND_TRUNC, seed: int = 0,
                  call: Optional[int] = None):
    """cuda/kernels.py:79-94.  x_ / w_ receive the quantized operands (allocate them with `alloc_int8`)."""
    assert x.is_cuda and w.is_cuda and (bias is None or bias.is_cuda)
    assert x.size(1) == w.size(1), "x and w must have the same number of columns"
    out_fp = torch.empty((x.size(0), w.size(0)), dtype=torch.float32, device=x.device)
    scale_out = torch.zeros_like(scaleX) if isReduce else torch.Tensor()
    bias = torch.Tensor() if bias is None else bias
    if mode == ROUND_STOCHASTIC and call is None:
        call = next_call()
        next_call()  # the weight draws from call + 1
    cuda_kernels.QGEMM_forward(out_fp, x, x_, w, w_, bias, scale_out, scaleX, scaleW, mode, seed, call or 0)
    return (out_fp, scale_out) if isReduce else out_fp


def QGEMM_backward(dY, X, W, scaledY, scaleX, scaleW, X_need=True, W_need=True, dx_row_scale=None):
    """cuda/kernels.py:97-111.  dx_row_scale (optional, [M]) multiplies row r of dX in the GEMM epilogue."""
    assert scaledY.is_cuda and dY.is_cuda
    dX, dW = None, None
    if X_need:
        assert W.is_cuda and scaleW.is_cuda
        dX = torch.empty(X.shape, dtype=torch.float32, device=X.device)
        cuda_kernels.QGEMM_backward_gradX(dX, dY, W, scaledY, scaleW, dx_row_scale)
    if W_need:
        assert X.is_cuda and scaleX.is_cuda
        dW = torch.empty(W.shape, dtype=torch.float32, device=X.device)
        cuda_kernels.QGEMM_backward_gradW(dW, dY, X, scaledY, scaleX)
    return dX, dW


def transpose_quant(data, scale):
    """cuda/kernels.py:114-119: fp32 [E,H,D] -> int8 [H,D,E]."""
    assert data.ndim == 3
    nrow = data.size(0)
    ncol = data.numel() // nrow
    data_ = cuda_kernels.transpose_quant(data, scale, nrow, ncol)
    return data_.reshape((data.size(1), data.size(2), nrow))


def multi_cusparse_SPMM(g, N, E_T, scale, reverse=False):
    """cuda/kernels.py:122-136.  E_T is int8 [H, 1, E] in edge-id order, as produced by `transpose_quant`; the
    per-slot permutation by edge_ids that the reference performs with index_select happens inside the kernel."""
    assert E_T.ndim == 3 and N.ndim == 3, "E and N must be 3D tensors"
    assert E_T.size(1) == 1, "Cannot broadcast E"
    indptr, indices, edge_ids = _bundle(g, reverse)
    E = E_T.reshape(E_T.shape[0], -1).t().contiguous()  # [E, H]
    return _u_mul_e_spmm(indptr, indices, edge_ids, N, E, scale, _schedule(g, reverse))


def spmm_u_mul_e_int8(g, N, E, scale, reverse=False):
    """Same product with the edge weights given as int8 [E, H] in edge-id order (no transposed copy)."""
    indptr, indices, edge_ids = _bundle(g, reverse)
    return _u_mul_e_spmm(indptr, indices, edge_ids, N, E.reshape(E.shape[0], -1), scale, _schedule(g, reverse))


def incidence_SPMM(g, E, scaleE, reverse=False):
    """cuda/kernels.py:139-152: sums int8 edge features into their destination (or source, if reverse) nodes."""
    assert E.is_cuda and scaleE.is_cuda
    indptr, _, edge_ids = _bundle(g, reverse)
    out_shape = (g.num_nodes(),) + E.shape[1:]
    dim = E.numel() // E.size(0)
    out = torch.empty((g.num_nodes(), dim), dtype=torch.float32, device=E.device)
    _incidence_spmm(out, indptr, edge_ids, E, scaleE, _schedule(g, reverse))
    return out.view(out_shape)


def csr_SPMM(g, N, scaleN, reverse=False, row_scale=None, bias=None, relu=False, out_absmax=None):
    """cuda/kernels.py:154-165; the keyword arguments fuse out = act(out * row_scale[:,None] + bias)."""
    indptr, indices, _ = g.adj_csr if reverse else g.adj_csc
    sched = _schedule(g, reverse)
    out_shape = (g.num_nodes(),) + N.shape[1:]
    dim = N.numel() // N.size(0)
    out = torch.empty((g.num_nodes(), dim), dtype=torch.float32, device=N.device)
    hub = getattr(g, "_hubs", {}).get("csr" if reverse else "csc")
    if hub is not None and N.dim() >= 2 and N.stride(0) % 16 == 0 and N.stride(0) == _round_up(dim, 16):
        # dense hub block on the tensor cores + the edges outside it through the gather kernels
        indptr, indices, sched = hub.indptr, hub.indices, hub.schedule
    _csr_spmm(out, indptr, indices, N, scaleN, sched, 1, row_scale, bias, relu, out_absmax)
    return out.view(out_shape)


def multi_cusparse_SPMV(g, N_T, E_T, scale, reverse=False):
    """cuda/kernels.py:167-178 forwards to multi_cusparse_SPMM in the reference; same here."""
    return multi_cusparse_SPMM(g, N_T, E_T, scale, reverse)


def _scale_word(device, want: bool):
    return torch.zeros(1, dtype=torch.float32, device=device) if want else None


def gat_edge_softmax(g, elq, erq, sl, sr, slope: float = 0.2, want_scale: bool = False):
    """Fused u_add_v -> LeakyReLU -> edge softmax over incoming edges; returns fp32 [E, H] in edge-id order (and,
    with want_scale, max|a|/127 from the kernel's epilogue)."""
    indptr, indices, edge_ids = _bundle(g, False)
    h = elq.shape[1]
    elq = elq.reshape(elq.shape[0], -1).contiguous()
    erq = erq.reshape(erq.shape[0], -1).contiguous()
    a = torch.empty((g.num_edges(), h), dtype=torch.float32, device=elq.device)
    sa = _scale_word(elq.device, want_scale)
    with torch.cuda.device(elq.device):
        sched = _schedule(g, False)
        order = sched.row_order if sched is not None else None
        check(lib.tango_gat_edge_softmax(_p(indptr), _p(indices), _p(edge_ids), _p(order),
                                         sched.n_block_rows if sched is not None else 0, g.num_nodes(), _p(elq), _p(erq), h,
                                         _p(sl), _p(sr), float(slope), _p(a), _p(sa), _stream()), "gat_edge_softmax")
    launch_counter[0] += 1
    return (a, sa) if want_scale else a


def gat_edge_softmax_bwd(g, elq, erq, sl, sr, a, da, slope: float = 0.2, want_scale: bool = False):
    """Gradient of `gat_edge_softmax` with respect to the edge logits (before the LeakyReLU); fp32 [E, H] (and, with
    want_scale, max|dz|/127)."""
    indptr, indices, edge_ids = _bundle(g, False)
    h = elq.shape[1]
    elq = elq.reshape(elq.shape[0], -1).contiguous()
    erq = erq.reshape(erq.shape[0], -1).contiguous()
    a, da = a.reshape(-1, h).contiguous(), da.reshape(-1, h).contiguous()
    dz = torch.empty_like(a)
    sdz = _scale_word(elq.device, want_scale)
    with torch.cuda.device(elq.device):
        sched = _schedule(g, False)
        order = sched.row_order if sched is not None else None
        check(lib.tango_gat_edge_softmax_bwd(_p(indptr), _p(indices), _p(edge_ids), _p(order),
                                             sched.n_block_rows if sched is not None else 0, g.num_nodes(), _p(elq), _p(erq), h,
                                             _p(sl), _p(sr), float(slope), _p(a), _p(da), _p(dz), _p(sdz), _stream()),
              "gat_edge_softmax_bwd")
    launch_counter[0] += 1
    return (dz, sdz) if want_scale else dz


def _gat_rows(g):
    sched = _schedule(g, False)
    order = sched.row_order if sched is not None else None
    return order, (sched.n_block_rows if sched is not None else 0)


def gat_edge_softmax_stats(g, elq, erq, sl, sr, slope: float = 0.2):
    """Step 1 of the attention weights without an fp32 copy: per-row softmax statistics (m, inv) [N, H] and the int8
    scale of the weights, max|a| / 127."""
    indptr, indices, _ = _bundle(g, False)
    h = elq.shape[1]
    elq, erq = elq.reshape(elq.shape[0], -1).contiguous(), erq.reshape(erq.shape[0], -1).contiguous()
    m = torch.empty((g.num_nodes(), h), dtype=torch.float32, device=elq.device)
    inv = torch.empty_like(m)
    sa = torch.zeros(1, dtype=torch.float32, device=elq.device)
    order, nb = _gat_rows(g)
    with torch.cuda.device(elq.device):
        check(lib.tango_gat_edge_softmax_stats(_p(indptr), _p(indices), _p(order), nb, g.num_nodes(), _p(elq), _p(erq),
                                               h, _p(sl), _p(sr), float(slope), _p(m), _p(inv), _p(sa), _stream()),
              "gat_edge_softmax_stats")
    launch_counter[0] += 1
    return m, inv, sa


def gat_edge_softmax_quantized(g, elq, erq, sl, sr, m, inv, sa, slope: float = 0.2, mode: int = ROUND_NEAREST,
                               seed: int = 0, call: int = 0) -> torch.Tensor:
    """Step 2: the int8 attention weights [E, H] in edge-id order, written once."""
    indptr, indices, edge_ids = _bundle(g, False)
    h = elq.shape[1]
    elq, erq = elq.reshape(elq.shape[0], -1).contiguous(), erq.reshape(erq.shape[0], -1).contiguous()
    aq = torch.empty((g.num_edges(), h), dtype=torch.int8, device=elq.device)
    order, nb = _gat_rows(g)
    with torch.cuda.device(elq.device):
        check(lib.tango_gat_edge_softmax_quantized(_p(indptr), _p(indices), _p(edge_ids), _p(order), nb, g.num_nodes(),
                                                   _p(elq), _p(erq), h, _p(sl), _p(sr), float(slope), _p(m), _p(inv),
                                                   _p(sa), _p(aq), mode, seed, call, _p(config.step_counter()),
                                                   _stream()), "gat_edge_softmax_quantized")
    launch_counter[0] += 1
    return aq


def gat_edge_softmax_bwd_stats(g, elq, erq, sl, sr, m, inv, da, slope: float = 0.2):
    """Gradient with respect to the edge logits, the weights recomputed from the statistics; returns (dz [E, H] fp32,
    max|dz| / 127)."""
    indptr, indices, edge_ids = _bundle(g, False)
    h = elq.shape[1]
    elq, erq = elq.reshape(elq.shape[0], -1).contiguous(), erq.reshape(erq.shape[0], -1).contiguous()
    da = da.reshape(-1, h).contiguous()
    dz = torch.empty_like(da)
    sdz = torch.zeros(1, dtype=torch.float32, device=elq.device)
    order, nb = _gat_rows(g)
    with torch.cuda.device(elq.device):
        check(lib.tango_gat_edge_softmax_bwd_stats(_p(indptr), _p(indices), _p(edge_ids), _p(order), nb, g.num_nodes(),
                                                   _p(elq), _p(erq), h, _p(sl), _p(sr), float(slope), _p(m), _p(inv),
                                                   _p(da), _p(dz), _p(sdz), _stream()), "gat_edge_softmax_bwd_stats")
    launch_counter[0] += 1
    return dz, sdz


def edge_softmax_fwd(g, z: torch.Tensor, zmul: float = 1.0, want_scale: bool = False):
    """Softmax of fp32 edge scores z [E, H, ...] (times zmul) over the incoming edges of every destination; the
    reference calls dgl.ops.edge_softmax (evaluation/test_HGT.py:60).  Returns fp32 of z's shape."""
    assert z.is_cuda and z.dtype == torch.float32
    indptr, _, edge_ids = _bundle(g, False)
    z2 = z.reshape(z.shape[0], -1).contiguous()
    h = z2.shape[1]
    assert z2.shape[0] == g.num_edges(), "one score row per edge"
    if h > 8:
        raise ValueError("edge_softmax: at most 8 heads")
    a = torch.empty_like(z2)
    sa = _scale_word(z.device, want_scale)
    with torch.cuda.device(z.device):
        sched = _schedule(g, False)
        order = sched.row_order if sched is not None else None
        check(lib.tango_edge_softmax(_p(indptr), _p(edge_ids), _p(order),
                                     sched.n_block_rows if sched is not None else 0, g.num_nodes(), _p(z2), h,
                                     float(zmul), _p(a), _p(sa), _stream()), "edge_softmax")
    launch_counter[0] += 1
    return (a.view(z.shape), sa) if want_scale else a.view(z.shape)


def edge_softmax_bwd(g, a: torch.Tensor, da: torch.Tensor, zmul: float = 1.0, want_scale: bool = False):
    """Gradient of `edge_softmax_fwd` with respect to z."""
    indptr, _, edge_ids = _bundle(g, False)
    a2 = a.reshape(a.shape[0], -1).contiguous()
    da2 = da.reshape(a2.shape).contiguous()
    h = a2.shape[1]
    dz = torch.empty_like(a2)
    sdz = _scale_word(a.device, want_scale)
    with torch.cuda.device(a.device):
        sched = _schedule(g, False)
        order = sched.row_order if sched is not None else None
        check(lib.tango_edge_softmax_bwd(_p(indptr), _p(edge_ids), _p(order),
                                         sched.n_block_rows if sched is not None else 0, g.num_nodes(), h, float(zmul),
                                         _p(a2), _p(da2), _p(dz), _p(sdz), _stream()), "edge_softmax_bwd")
    launch_counter[0] += 1
    return (dz.view(a.shape), sdz) if want_scale else dz.view(a.shape)


def relu_grad_stats(g: torch.Tensor, y: torch.Tensor, row_scale: Optional[torch.Tensor] = None,
                    want_colsum: bool = True):
    """(scale, column sums or None) of the masked gradient (y > 0 ? g : 0); the scale includes row_scale."""
    g, rows, cols, ldg = _matrix(g)
    y, _, _, ldy = _matrix(y)
    scale = torch.empty(1, dtype=torch.float32, device=g.device)
    colsum = torch.empty(cols, dtype=torch.float32, device=g.device) if want_colsum else None
    nbytes = lib.tango_relu_grad_stats_scratch_bytes(rows, cols) if want_colsum else 0
    scratch = torch.empty(max(nbytes, 4), dtype=torch.uint8, device=g.device)
    with torch.cuda.device(g.device):
        check(lib.tango_relu_grad_stats(_p(g), ldg, _p(y), ldy, rows, cols, _p(row_scale), _p(scale), _p(colsum),
                                        _p(scratch), nbytes, _stream()), "relu_grad_stats")
    launch_counter[0] += 2 if want_colsum else 1
    return scale, colsum


def relu_grad_quant(g: torch.Tensor, y: torch.Tensor, row_scale: Optional[torch.Tensor], scale: torch.Tensor,
                    mode: int = ROUND_NEAREST, seed: int = 0, call: int = 0) -> torch.Tensor:
    """int8 of (y > 0 ? g : 0) * row_scale / scale, rows padded to 16 bytes."""
    g, rows, cols, ldg = _matrix(g)
    y, _, _, ldy = _matrix(y)
    q = alloc_int8((rows, cols), g.device)
    with torch.cuda.device(g.device):
        check(lib.tango_quantize_relu_grad(_p(g), ldg, _p(y), ldy, rows, cols, _p(row_scale), _p(scale), _p(q),
                                           q.stride(0), mode, seed, call, _p(config.step_counter()), _stream()),
              "quantize_relu_grad")
    launch_counter[0] += 1
    return q


def relu_grad_quantize(g: torch.Tensor, y: torch.Tensor, row_scale: Optional[torch.Tensor] = None,
                       want_colsum: bool = True, mode: int = ROUND_NEAREST, seed: int = 0, call: int = 0):
    """For the backward pass of y = relu(.): returns (int8 of (y > 0 ? g : 0) * row_scale / scale, scale, column sums
    of the masked gradient or None) without materialising the masked gradient."""
    scale, colsum = relu_grad_stats(g, y, row_scale, want_colsum)
    return relu_grad_quant(g, y, row_scale, scale, mode, seed, call), scale, colsum
