import os
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def golden():
    path = os.path.join(ROOT, "tests", "golden", "decode_path_golden.npz")
    with np.load(path) as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def orc():
    import oracle

    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def cuda():
    """torch with a CUDA device and the library loaded; GPU tests fail (not skip) if either is missing."""
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from nve_b200 import _ffi

    _ffi.load()
    torch.cuda.set_device(0)
    return torch
