"""tango_b200: B200-native (sm_100a) kernels behind Tango's quantized GNN-training operator API.

Modules mirror the reference's `cuda/` package: `kernels`, `QLinear`, `SPMM`, `SDDMM`, `util`.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library has not been built)
from . import config, graph, kernels, util  # noqa: F401
from .QLinear import QLinear, Qlinear_func, Qlinear_func_reduce, QgemmNT_func  # noqa: F401
from .SDDMM import sddmm_u_add_v, sddmm_u_dot_v  # noqa: F401
from .SPMM import spmm_copy_u, spmm_u_mul_e  # noqa: F401
from .util import graph_preprocess  # noqa: F401

__version__ = "0.1.0"
