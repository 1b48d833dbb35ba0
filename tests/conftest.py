import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def oracle32():
    from oracle.nrs_oracle import Oracle
    return Oracle("f32")


@pytest.fixture(scope="session")
def oracle64():
    from oracle.nrs_oracle import Oracle
    return Oracle("f64")


@pytest.fixture(scope="session")
def nrs_lib():
    """The shared library, built in-tree if absent (nvcc cross-compiles without a GPU)."""
    from neuralrs_b200 import _lib
    if not _lib.LIB_PATH.exists():
        from neuralrs_b200 import build
        build.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def gpu_ctx(nrs_lib):
    """Default device context; GPU tests fail (not skip) when the device or library is unusable."""
    from neuralrs_b200 import cuda
    return cuda.default_context()


def rel_l2(a, ref):
    a = np.asarray(a, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    d = np.linalg.norm(a - ref)
    n = np.linalg.norm(ref)
    return d / n if n > 0 else d


def max_rel(a, ref):
    """max |a-ref| / (|ref| + 1e-6*max|ref|): the elementwise form of the 1e-4 bar."""
    a = np.asarray(a, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    scale = np.abs(ref).max() if ref.size else 0.0
    return float(np.max(np.abs(a - ref) / (np.abs(ref) + 1e-6 * scale + 1e-30))) if ref.size else 0.0
