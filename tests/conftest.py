import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    # A GPU test that silently skips would hide a missing device; fail instead
    # unless the run deselected gpu tests with -m "not gpu".
    pass


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "reference_oracle_outputs.npz")
    return np.load(path, allow_pickle=False)


@pytest.fixture(scope="session")
def golden_kv_compress():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "reference_kv_compress_outputs.npz")
    return np.load(path, allow_pickle=False)
