import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def native_lib():
    """The C-ABI library, built in-tree if stale. Never replaced by a fallback."""
    from ultra_ep_b200 import build, capi

    build.build_native()
    return capi.lib()


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    torch.cuda.set_device(0)
    return torch.device("cuda", 0)
