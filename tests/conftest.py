import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "lif_golden.npz"))


@pytest.fixture(scope="session")
def config1_digest():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "lif_config1_digest.npz"))


@pytest.fixture(scope="session")
def built_lib():
    """Build (if stale) and return the path of libsnn_b200.so."""
    from snn_gpu_training_bptt_b200 import build
    return build.build()
