"""ctypes binding of libtango_b200.so (the C ABI declared in include/tango_b200.h).

The library is prebuilt in-tree (python tango_b200/build.py); there is no fallback implementation: if the shared
object is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TANGO_B200_LIB") or os.path.join(_HERE, "lib", "libtango_b200.so")

TANGO_OK = 0
TANGO_EALIGN = -2
TANGO_ETIMEOUT = -4
ROUND_TRUNC, ROUND_NEAREST, ROUND_STOCHASTIC = 0, 1, 2
OPS = {"add": 0, "sub": 1, "mul": 2, "div": 3}


class SpmmPlan(Structure):
    _fields_ = [
        ("units", c_void_p),
        ("n_units", c_int64),
        ("heavy_rows", c_void_p),
        ("n_heavy", c_int64),
        ("ws", c_void_p),
        ("ws_ld", c_int64),
        ("split_threshold", c_int32),
        ("row_order", c_void_p),
        ("n_long_rows", c_int64),
        ("dense_a", c_void_p),
        ("dense_n_tiles", c_int64),
        ("dense_units", c_void_p),
        ("dense_n_units", c_int64),
        ("dense_rows", c_int64),
        ("dense_cols", c_void_p),
        ("dense_n_cols", c_int64),
        ("dense_b", c_void_p),
        ("dense_status", c_void_p),
        ("n_skip_rows", c_int64),
    ]


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build the CUDA library first with `python tango_b200/build.py` "
        "(there is no CPU or PyTorch fallback for these operators)")

lib = ctypes.CDLL(LIB_PATH)

P = c_void_p
_SIGS = {
    "tango_version": ([], c_int),
    "tango_strerror": ([c_int], c_char_p),
    "tango_last_cuda_error": ([], c_int),
    "tango_absmax_scale": ([P, c_int64, c_int64, c_int64, P, P, P], c_int),
    "tango_quantize": ([P, c_int64, c_int64, c_int64, P, P, P, c_int64, c_int, c_uint64, c_uint64, P, P], c_int),
    "tango_quantize_transpose": ([P, c_int64, c_int64, P, P, P], c_int),
    "tango_relu_grad_stats_scratch_bytes": ([c_int64, c_int64], c_int64),
    "tango_relu_grad_stats": ([P, c_int64, P, c_int64, c_int64, c_int64, P, P, P, P, c_int64, P], c_int),
    "tango_quantize_relu_grad": ([P, c_int64, P, c_int64, c_int64, c_int64, P, P, P, c_int64, c_int, c_uint64,
                                  c_uint64, P, P], c_int),
    "tango_qgemm_dw_workspace_bytes": ([c_int64, c_int64], c_int64),
    "tango_qgemm_nt": ([P, c_int64, P, c_int64, c_int64, c_int64, c_int64, P, P, P, P, c_int64, P, P, P], c_int),
    "tango_qgemm_forward": ([P, c_int64, P, P, c_int64, c_int64, c_int64, c_int64, P, P, P, c_int64, P, c_int64, P, P,
                             c_int64, P, c_int, c_uint64, c_uint64, P, P, P], c_int),
    "tango_qgemm_dx": ([P, c_int64, P, c_int64, c_int64, c_int64, c_int64, P, P, P, P, c_int64, P, P], c_int),
    "tango_qgemm_dw": ([P, c_int64, P, c_int64, c_int64, c_int64, c_int64, P, P, P, c_int64, P, c_int64, P, P], c_int),
    "tango_qgemm_dw_noalloc": ([P, c_int64, P, c_int64, c_int64, c_int64, c_int64, P, P, P, c_int64, P, P], c_int),
    "tango_qgemm_dw_noalloc_max_elems": ([], c_int64),
    "tango_spmm_copy_u": ([P, P, c_int64, c_int, P, c_int64, c_int64, P, P, P, c_int, P, c_int64, P,
                           POINTER(SpmmPlan), P], c_int),
    "tango_spmm_u_mul_e": ([P, P, P, c_int64, P, c_int64, c_int, c_int, P, P, P, c_int64, POINTER(SpmmPlan), P], c_int),
    "tango_spmm_incidence": ([P, P, c_int64, P, c_int64, c_int64, P, P, c_int64, POINTER(SpmmPlan), P], c_int),
    "tango_sddmm_dot": ([P, P, c_int64, P, c_int64, P, c_int64, c_int, c_int, P, P, P, P, P], c_int),
    "tango_sddmm_dot_rows": ([P, P, P, c_int64, P, c_int64, P, c_int64, c_int, c_int, P, P, P, P, P, P], c_int),
    "tango_sddmm_elementwise": ([c_int, P, P, c_int64, P, c_int64, P, c_int64, c_int64, P, P, P, P, P], c_int),
    "tango_gat_edge_softmax": ([P, P, P, P, c_int64, c_int64, P, P, c_int, P, P, c_float, P, P, P], c_int),
    "tango_gat_edge_softmax_bwd": ([P, P, P, P, c_int64, c_int64, P, P, c_int, P, P, c_float, P, P, P, P, P], c_int),
    "tango_gat_edge_softmax_stats": ([P, P, P, c_int64, c_int64, P, P, c_int, P, P, c_float, P, P, P, P], c_int),
    "tango_gat_edge_softmax_quantized": ([P, P, P, P, c_int64, c_int64, P, P, c_int, P, P, c_float, P, P, P, P, c_int,
                                          c_uint64, c_uint64, P, P], c_int),
    "tango_gat_edge_softmax_bwd_stats": ([P, P, P, P, c_int64, c_int64, P, P, c_int, P, P, c_float, P, P, P, P, P, P],
                                         c_int),
    "tango_quantize_push": ([P, c_int64, c_int64, c_int64, P, P, P, c_int, c_int64, c_int64, c_int, c_uint64, c_uint64,
                             P, P], c_int),
    "tango_quantize_relu_grad_push": ([P, c_int64, P, c_int64, c_int64, c_int64, P, P, P, c_int, c_int64, c_int64, c_int,
                                       c_uint64, c_uint64, P, P], c_int),
    "tango_peer_alloc": ([c_int64, P, P], c_int),
    "tango_peer_open": ([P, P], c_int),
    "tango_peer_close": ([P], c_int),
    "tango_peer_free": ([P], c_int),
    "tango_enable_peer_access": ([c_int], c_int),
    "tango_peer_sync": ([P, c_int, c_int, P, P, P, P, c_int64, P], c_int),
    "tango_edge_softmax": ([P, P, P, c_int64, c_int64, P, c_int, c_float, P, P, P], c_int),
    "tango_edge_softmax_bwd": ([P, P, P, c_int64, c_int64, c_int, c_float, P, P, P, P, P], c_int),
}
for _name, (_args, _res) in _SIGS.items():
    if not hasattr(lib, _name):
        raise ImportError(f"{LIB_PATH} is stale (no symbol {_name}): rebuild it with `python tango_b200/build.py`")
    _fn = getattr(lib, _name)
    _fn.argtypes = _args
    _fn.restype = _res

EXPORTED = tuple(_SIGS)


class TangoError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != TANGO_OK:
        msg = lib.tango_strerror(rc).decode()
        extra = f" (cudaError {lib.tango_last_cuda_error()})" if rc == -3 else ""
        raise TangoError(f"{what}: {msg}{extra}")
