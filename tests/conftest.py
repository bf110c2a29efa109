import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def dev():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True, scope="module")
def _no_kernel_wait_timed_out():
    """After every test module that ran on a GPU: none of the tcgen05 kernels' bounded waits may have given up.  A wait
    that times out leaves wrong outputs behind only for the launch it happened in, which a later assertion can miss."""
    yield
    import torch

    if torch.cuda.is_available():
        import mlx_flashattention_steel_b200 as fa

        assert fa.kernel_status() == 0, "a bounded wait inside a tcgen05 kernel timed out during this module"
