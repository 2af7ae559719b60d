"""Shared pytest configuration: the ``gpu`` marker, import paths and seeding."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "mamba-ascendc_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(autouse=True)
def fixed_seed():
    """Same convention as the reference's tests/conftest.py:19-25: every test starts from seed 42."""
    import torch

    torch.manual_seed(42)
    yield
