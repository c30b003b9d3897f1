import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session", autouse=True)
def _library_built():
    """The C-ABI library must exist before any test imports the package (there is no fallback to test instead)."""
    import __graft_entry__
    __graft_entry__.build()


@pytest.fixture()
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


# Problem shapes the reference's correctness tests sweep (tests/conftest.py:40-60 of the reference tree).
STANDARD_DIMS = [(128, 128, 128), (256, 256, 256), (512, 512, 512), (1024, 1024, 1024), (384, 640, 256)]
EDGE_CASE_DIMS = [(8, 128, 256), (15, 17, 512), (19, 13, 512), (128, 64, 12), (16, 16, 4096), (32, 32, 8192),
                  (1, 256, 512), (257, 129, 200)]
