import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")
    # make sure the prebuilt library exists before any test imports the package (nvcc cross-compiles without a GPU)
    # the build script is loaded by path: importing the package itself needs an up-to-date library
    import importlib.util
    spec = importlib.util.spec_from_file_location("_tango_build", os.path.join(ROOT, "tango_b200", "build.py"))
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    build.build()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
