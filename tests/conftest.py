import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(params=["rowmajor", "transposed"])
def wgrad_dataflow(request):
    """Runs a module test under both weight-gradient dataflows: operands read row-major by the GEMM (default) and the
    reference's padded transposes (FP8GMM_WGRAD=transposed)."""
    from fp8_gmm_b200 import backend

    saved = backend.WGRAD_ROWMAJOR
    backend.WGRAD_ROWMAJOR = request.param == "rowmajor"
    yield request.param
    backend.WGRAD_ROWMAJOR = saved
