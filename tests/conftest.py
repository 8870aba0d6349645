import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device and the built sm_100a library")


@pytest.fixture(scope="session")
def reference_fixtures():
    """The reference project's saved block/step fixtures as raw tensor trees."""
    return torch.load(GOLDEN / "reference_fixtures.pt", map_location="cpu", weights_only=True)


@pytest.fixture(scope="session")
def reference_outputs():
    """Outputs of the reference's functions on seeded NVFP4 inputs (raw tensor trees)."""
    return torch.load(GOLDEN / "reference_outputs.pt", map_location="cpu", weights_only=True)


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
