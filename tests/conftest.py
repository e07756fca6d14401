"""pytest configuration: the ``gpu`` marker and the import path of the repo root."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (compute capability 10.x)")


@pytest.fixture(scope="session")
def native_lib():
    """The C-ABI library, built in-tree if it is stale or missing."""
    from chord_b200 import _lib, build

    build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    from chord_b200 import build

    build.build()
    return torch.device("cuda:0")
