import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    """The three fixture archives produced by tests/golden/make_golden.py from the reference."""
    import numpy as np
    here = os.path.join(ROOT, "tests", "golden")
    return {name: np.load(os.path.join(here, name + ".npz"))
            for name in ("metadata", "convert", "matmul")}
