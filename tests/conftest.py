import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def lib():
    """The built C-ABI library; building is part of the session when the .so is absent."""
    import boat_b200
    from boat_b200 import capi
    if not os.path.exists(capi.lib_path()):
        boat_b200.build()
    return capi.load()


@pytest.fixture(scope="session")
def gpu_lib(lib):
    """The library on a machine with a GPU; a GPU test without a device is an error, not a skip."""
    assert lib.boat_cuda_device_count() > 0, "GPU test collected on a machine without a CUDA device"
    rc = lib.boat_cuda_init(-1)
    assert rc == 0, lib.boat_cuda_last_error()
    return lib


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "attention_golden.npz"))
