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
    """Runs a module test under both backward dataflows: operands read as they lie by the GEMMs (default: row-major
    activations for wgrad, forward weights for dgrad) and the reference's transposes (FP8GMM_WGRAD=transposed,
    FP8GMM_DGRAD=transposed)."""
    from fp8_gmm_b200 import backend

    saved = backend.WGRAD_ROWMAJOR, backend.DGRAD_KN
    backend.WGRAD_ROWMAJOR = backend.DGRAD_KN = request.param == "rowmajor"
    yield request.param
    backend.WGRAD_ROWMAJOR, backend.DGRAD_KN = saved
