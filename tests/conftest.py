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
def tb():
    """One library handle on cuda:0 for the whole GPU session."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ter_b200 import TerB200
    h = TerB200(0)
    yield h
    assert h.device_status() == 0
    h.close()
