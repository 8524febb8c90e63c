"""Compiles the reference's own CUDA sources, where they lie, into oracle/_ref/tango_ref.so (test infrastructure).

Sources taken from the Tango checkout (never copied): cuda/src/quantization.cu, SDDMM.cu, QGEMM_backward.cu and
SPMM.cu, with the reference's own nvcc flags (-O3 --use_fast_math, cuda/kernels.py:12-16), plus the binding
oracle/ref_binding.cpp.  cuda/src/QGEMM_forward.cu is left out: it is written against the CUTLASS 2.x kernel
concept and does not compile against the CUTLASS headers on this image.  Needs the torch C++ headers and a CUTLASS
header tree (the one vendored inside the flashinfer wheel).

    python oracle/build_ref.py [/path/to/Tango]      # build (about five minutes)

`load()` imports the built module; it never builds.  The module needs a CUDA device to do anything useful; the
fixtures under tests/golden/ that pin the CPU oracle were produced with it by tests/golden/make_ref_fixtures.py.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
NAME = "tango_ref"
SOURCES = ["quantization.cu", "SDDMM.cu", "QGEMM_backward.cu", "SPMM.cu"]
DEFAULT_REFERENCE_ROOT = os.path.join(os.sep, "root", "reference")    # where the build container mounts the checkout


def _cutlass_include():
    site = sysconfig.get_paths()["purelib"]
    for rel in ("flashinfer/data/cutlass", "tilelang/3rdparty/cutlass"):
        root = os.path.join(site, rel)
        if os.path.isdir(os.path.join(root, "include", "cutlass")):
            return [os.path.join(root, "include"), os.path.join(root, "tools", "util", "include")]
    raise RuntimeError("no CUTLASS header tree found")


def module_path():
    for f in sorted(os.listdir(OUT_DIR)) if os.path.isdir(OUT_DIR) else []:
        if f.startswith(NAME) and f.endswith(".so"):
            return os.path.join(OUT_DIR, f)
    return None


def build(reference_root: str = DEFAULT_REFERENCE_ROOT, verbose: bool = True):
    src_dir = os.path.join(reference_root, "cuda", "src")
    if not os.path.isdir(src_dir):
        raise FileNotFoundError(f"no reference checkout at {reference_root}")
    os.makedirs(OUT_DIR, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", "5")
    from torch.utils.cpp_extension import load
    load(name=NAME, sources=[os.path.join(HERE, "ref_binding.cpp")] + [os.path.join(src_dir, s) for s in SOURCES],
         extra_cflags=["-O3", "-DTANGO_REF_WITH_SPMM"],
         extra_cuda_cflags=["-O3", "--use_fast_math", "--generate-line-info"],
         extra_ldflags=["-lcusparse"], extra_include_paths=_cutlass_include() + [src_dir],
         build_directory=OUT_DIR, verbose=verbose, is_python_module=False)
    return module_path()


def load():
    """The built module, or None when oracle/_ref holds none."""
    path = module_path()
    if path is None:
        return None
    import torch  # noqa: F401  (the module links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE_ROOT))
