"""tango_b200: B200-native (sm_100a) kernels behind Tango's quantized GNN-training operator API.

Modules mirror the reference's `cuda/` package: `kernels`, `QLinear`, `SPMM`, `SDDMM`, `util`.
"""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library has not been built)
from . import config, graph, kernels, util  # noqa: F401
from .QLinear import QLinear, Qlinear_func, Qlinear_func_reduce, QgemmNT_func  # noqa: F401
from .SDDMM import sddmm_u_add_v, sddmm_u_dot_v  # noqa: F401
from .SPMM import spmm_copy_u, spmm_u_mul_e  # noqa: F401
from .util import graph_preprocess  # noqa: F401

__version__ = "0.2.0"


def install_as_cuda() -> None:
    """Makes this package importable under the name the reference's scripts use: after the call
    `import cuda`, `from cuda.kernels import *`, `from cuda.QLinear import QLinear`, `from cuda import SPMM, SDDMM,
    util` (evaluation/test_fuse.py:48-49, evaluation/SPMM_broadcast.py:15, evaluation/test_gcn.py:21-24) resolve to
    the SAME module objects as `tango_b200.*` -- one copy of every module, so settings made through either name
    (config.set_rounding, the call counters, the status words) are seen through both.  Registering only the
    top-level name would make `cuda.kernels` a second, independent copy of each submodule."""
    import importlib
    import sys
    sys.modules["cuda"] = sys.modules[__name__]
    # looked up by module name: the package attribute `QLinear` is the class, not the module
    for name in ("kernels", "QLinear", "SPMM", "SDDMM", "util", "config", "graph", "_lib", "gnn", "dist", "peer"):
        sys.modules[f"cuda.{name}"] = importlib.import_module(f"{__name__}.{name}")
