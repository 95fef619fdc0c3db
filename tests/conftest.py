import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (sm_100a)")


def rel_err(new, ref):
    """max|new - ref| / max(max|ref|, 1e-12), the error metric used for every parity check."""
    new = new.detach().double().cpu()
    ref = ref.detach().double().cpu()
    assert new.shape == ref.shape, (new.shape, ref.shape)
    if ref.numel() == 0:
        return 0.0
    return float((new - ref).abs().max() / max(float(ref.abs().max()), 1e-12))


@pytest.fixture(scope="session")
def op_cases():
    return torch.load(os.path.join(GOLDEN, "op_cases.pt"), weights_only=False)


@pytest.fixture(scope="session")
def model_cases():
    return torch.load(os.path.join(GOLDEN, "model_cases.pt"), weights_only=False)


@pytest.fixture(scope="session")
def regression_case():
    return torch.load(os.path.join(GOLDEN, "regression_2_3_5.pt"), weights_only=False)


@pytest.fixture(scope="session")
def layer_norm_cases():
    return torch.load(os.path.join(GOLDEN, "layer_norm_cases.pt"), weights_only=False)
