import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def oracle_lib():
    from oracle import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def kernels():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from adrastea_b200 import GpuKernels
    return GpuKernels(0)
