import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from xpu_graph_b200 import lib

    L = lib.load()  # raises if the library is missing: GPU tests never run on a silent fallback
    assert L.xg_device_arch_ok(torch.cuda.current_device()) == 1, "kernels are built for sm_100a only"
    return torch.device("cuda", torch.cuda.current_device())
