import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def hm():
    """The product package; building it first if the shared library is missing."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("b200mlir_build", os.path.join(ROOT, "hexagon_mlir_b200", "build.py"))
    build = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(build)
    build.build_library()  # no-op when the library is newer than its sources
    import hexagon_mlir_b200
    return hexagon_mlir_b200


@pytest.fixture(scope="session")
def oracle():
    import oracle as _oracle
    _oracle.lib()
    return _oracle


def philox(seed):
    import numpy as np
    return np.random.Generator(np.random.Philox(seed))


def max_abs_rel(got, ref):
    """max|got - ref| / max|ref| — the 'max-abs-rel' error the tolerances are stated in."""
    import numpy as np
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = max(float(np.abs(ref).max()), 1e-30)
    return float(np.abs(got - ref).max()) / denom


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch
