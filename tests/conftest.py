import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    def load(name):
        return dict(np.load(os.path.join(GOLDEN, name)))

    return load


@pytest.fixture
def tc_from_256_rows():
    """Pins Linear layers to the tcgen05 kernels from 256 coefficient rows on (BF_B200_TC_MIN_ROWS=256, read at every
    call).  The default policy additionally keeps a layer on the FFMA kernels while its 64 x 64 tiles fit one wave, which
    covers the mid-sized cases (288-1152 rows) that the tensor-core tests use on purpose."""
    old = os.environ.get("BF_B200_TC_MIN_ROWS")
    os.environ["BF_B200_TC_MIN_ROWS"] = "256"
    yield
    if old is None:
        os.environ.pop("BF_B200_TC_MIN_ROWS", None)
    else:
        os.environ["BF_B200_TC_MIN_ROWS"] = old
