import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.port()
    return O


@pytest.fixture(scope="session")
def ops():
    """The product's Python mirror with the library initialised on cuda:0. GPU tests only."""
    import torch
    assert torch.cuda.is_available(), "GPU test selected without a CUDA device"
    torch.cuda.set_device(0)
    import rocm_hip_b200 as m
    assert m.gpu_ops_init("gpu_ops.co") == 0, "gpu_ops_init failed: the kernels are not loadable on this device"
    return m
