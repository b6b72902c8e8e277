import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def backend():
    """One library context on cuda:0 for the whole GPU session; fails loudly if the CUDA library is missing."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from inferi_b200.ops import Backend

    torch.cuda.set_device(0)
    b = Backend(0)
    yield b
    b.close()
