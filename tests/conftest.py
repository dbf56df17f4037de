"""pytest configuration: the `gpu` marker and shared fixtures.

`-m "not gpu"` runs on a machine without a GPU (oracle vs golden vectors, host logic,
ABI surface).  `-m gpu` needs a B200 and calls the CUDA kernels through the C ABI.
"""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "reference_vectors.npz")


@pytest.fixture(scope="session")
def fdl():
    """The kernel library binding; building it needs nvcc but no GPU."""
    from fast_dl_b200 import build, capi
    build.build_kernels()
    capi.lib()
    return capi


@pytest.fixture(scope="session")
def cuda(fdl):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    fdl.use_device(0)
    return torch
