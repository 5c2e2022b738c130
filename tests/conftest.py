import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")
    lib = os.path.join(ROOT, "vdcores_b200", "libvdcores_b200.so")
    if not os.path.exists(lib):
        # nvcc cross-compiles without a GPU; the product has no other code path
        subprocess.check_call([sys.executable, "-m", "vdcores_b200.build"], cwd=ROOT)


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
