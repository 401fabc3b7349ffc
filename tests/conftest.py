import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
for p in (ROOT, GOLDEN):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_sessionstart(session):
    """Compile the CUDA extension (nvcc cross-compiles without a GPU) and the C checker if they are
    missing or older than their sources, so that a fresh checkout can run the suite directly."""
    from permutohedral_encoding_b200 import build as ext_build
    ext_build.build()
    from oracle import permuto_oracle
    permuto_oracle.build()


def pytest_collection_modifyitems(config, items):
    # every test in a test_gpu_* / test_zz_* file needs the device even when the mark was forgotten
    for item in items:
        base = os.path.basename(str(item.fspath))
        if base.startswith("test_gpu_") and "gpu" not in item.keywords:
            item.add_marker(pytest.mark.gpu)


def densify(idx, val, shape):
    out = np.zeros(int(np.prod(shape)), np.float32)
    out[idx] = val
    return out.reshape(shape)


@pytest.fixture(scope="session")
def oracle():
    from oracle import permuto_oracle as po
    po.set_modes(1, 1)
    return po
