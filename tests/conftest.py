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
    from hexagon_mlir_b200 import build
    if not os.path.exists(build.LIB):
        build.build_library()
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
