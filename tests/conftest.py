import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def cuda():
    """torch with a CUDA device; GPU tests fail (not skip) when the device is missing."""
    import torch
    assert torch.cuda.is_available(), "GPU test run without a CUDA device"
    torch.cuda.set_device(0)
    return torch
