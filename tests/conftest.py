import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_index():
    import numpy as np
    return np.load(os.path.join(GOLDEN, "index_layer.npz"))


@pytest.fixture(scope="session")
def golden_cg():
    import numpy as np
    return np.load(os.path.join(GOLDEN, "cg_coefficients.npz"))


@pytest.fixture(scope="session")
def golden_layers():
    import numpy as np
    return np.load(os.path.join(GOLDEN, "layer_cases.npz"))
