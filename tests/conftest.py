import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import torch

    return torch.load(ROOT / "tests" / "golden" / "asynctp_golden.pt", weights_only=False)


@pytest.fixture(scope="session")
def golden_fp8():
    import torch

    return torch.load(ROOT / "tests" / "golden" / "asynctp_golden_fp8.pt", weights_only=False)
