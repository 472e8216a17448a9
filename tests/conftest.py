import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if os.fspath(ROOT) not in sys.path:
    sys.path.insert(0, os.fspath(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def clef_lib():
    """The C-ABI library, built in-tree if it is missing or stale (nvcc cross-compiles without a GPU)."""
    from aiis_clef_b200.build import build_library
    import aiis_clef_b200 as clef

    build_library()
    return clef.load()


@pytest.fixture(scope="session")
def cuda_dev():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    import aiis_clef_b200 as clef

    return clef.Device(0)
