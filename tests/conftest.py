"""Shared pytest configuration: makes the in-tree package importable and registers the `gpu` marker."""
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
PKG_DIR = REPO / "flash-linear-attention-npu_b200"
for p in (str(PKG_DIR), str(REPO)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (sm_100a) and the built kernel library")


@pytest.fixture(scope="session")
def lib():
    import fla_b200

    return fla_b200.load_library()
