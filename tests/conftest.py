import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def lib():
    """The CUDA library through the C ABI.  Built in-tree; never falls back to anything else."""
    from cute_mma_b200 import build, ops

    build.build()
    return ops.load_library()


@pytest.fixture(scope="session")
def cuda():
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch.device("cuda:0")


@pytest.fixture(scope="session")
def pair_build(lib):
    """True when the library was built with CTA pairs (ctas = 2, the default); a few features exist only there."""
    from cute_mma_b200 import ops

    return ops.kernel_info(lib)["oft"]["ctas"] == 2
