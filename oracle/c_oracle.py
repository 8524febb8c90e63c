"""NumPy-facing wrappers of the plain-C checker (oracle_c.c).  Test infrastructure only."""
from __future__ import annotations

import numpy as np

from . import build_c

_lib = None


def _l():
    global _lib
    if _lib is None:
        _lib = build_c.load()
    return _lib


def _p(a):
    return a.ctypes.data


def absmax_scale(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    return np.float32(_l().oc_absmax_scale(_p(x), x.size))


def quantize(x, scale, mode=1, seed=0, call=0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.empty(x.shape, dtype=np.int8)
    _l().oc_quantize(_p(x), x.size, float(scale), mode, seed, call, _p(q))
    return q


def igemm_nt(a, b):
    a, b = np.ascontiguousarray(a, np.int8), np.ascontiguousarray(b, np.int8)
    acc = np.empty((a.shape[0], b.shape[0]), dtype=np.int32)
    _l().oc_igemm_nt(_p(a), _p(b), a.shape[0], b.shape[0], a.shape[1], _p(acc))
    return acc


def spmm_copy_u(indptr, indices, nq, scale):
    indptr, indices = np.ascontiguousarray(indptr, np.int64), np.ascontiguousarray(indices, np.int64)
    nq2 = np.ascontiguousarray(nq.reshape(nq.shape[0], -1), np.int8)
    out = np.empty((len(indptr) - 1, nq2.shape[1]), dtype=np.float32)
    _l().oc_spmm_copy_u(_p(indptr), _p(indices), len(indptr) - 1, _p(nq2), nq2.shape[1], float(scale), _p(out))
    return out


def spmm_u_mul_e(indptr, indices, eids, nq, eq, scale):
    indptr, indices = np.ascontiguousarray(indptr, np.int64), np.ascontiguousarray(indices, np.int64)
    eids = None if eids is None else np.ascontiguousarray(eids, np.int64)
    nq, eq = np.ascontiguousarray(nq, np.int8), np.ascontiguousarray(eq, np.int8)
    _, h, d = nq.shape
    out = np.empty((len(indptr) - 1, h, d), dtype=np.float32)
    _l().oc_spmm_u_mul_e(_p(indptr), _p(indices), None if eids is None else _p(eids), len(indptr) - 1, _p(nq), h, d,
                         _p(eq), float(scale), _p(out))
    return out


def sddmm_dot(src, dst, uq, vq, su, sv):
    src, dst = np.ascontiguousarray(src, np.int64), np.ascontiguousarray(dst, np.int64)
    uq, vq = np.ascontiguousarray(uq, np.int8), np.ascontiguousarray(vq, np.int8)
    _, h, d = uq.shape
    out = np.empty((len(src), h), dtype=np.float32)
    _l().oc_sddmm_dot(_p(src), _p(dst), len(src), _p(uq), _p(vq), h, d, float(su), float(sv), _p(out))
    return out
