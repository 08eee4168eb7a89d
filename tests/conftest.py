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

    return np.load(os.path.join(ROOT, "tests", "golden", "dense_path.npz"))


def bf16(array):
    import torch

    return torch.from_numpy(array.copy()).view(torch.bfloat16)


def e4m3(array):
    import torch

    return torch.from_numpy(array.copy()).view(torch.float8_e4m3fn)


@pytest.fixture(scope="session")
def golden_sol():
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "sol_path.npz"))


@pytest.fixture(scope="session")
def golden_norm_rope():
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "norm_rope.npz"))


@pytest.fixture(scope="session")
def golden_matmul():
    """Inputs and reference ref_program outputs of the projection GEMMs (tests/golden/make_golden.py)."""
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "matmul.npz"))
