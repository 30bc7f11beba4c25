import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from katz_b200 import load_library
    load_library()   # a missing library is a failure, not a skip
    return torch.device("cuda:0")


@pytest.fixture(autouse=True, scope="module")
def _release_cached_device_memory():
    """The SDXL-size tests peak at tens of GB; hand the caching allocator's blocks back after every test module so that
    tests which start other processes on the same GPU find room."""
    yield
    import gc
    import torch
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        gc.collect()
        torch.cuda.empty_cache()
