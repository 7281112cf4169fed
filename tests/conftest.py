import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "decode_golden.npz")
    return dict(np.load(path))


@pytest.fixture(scope="session")
def prefill_golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "prefill_golden.npz")
    return dict(np.load(path))
