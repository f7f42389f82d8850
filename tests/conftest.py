import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import khq_oracle

    khq_oracle.build()
    khq_oracle.load()
    return khq_oracle


@pytest.fixture(scope="session")
def cuda_ops():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from bonsai_mojo_1bit_optimization_t4_cuda_b200 import build as _build
    from bonsai_mojo_1bit_optimization_t4_cuda_b200.ops import CudaOps

    if not _build.LIB_PATH.exists():
        _build.build()
    return CudaOps()
