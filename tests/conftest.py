import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def oracle():
    from oracle import loader
    loader.lib()
    return loader


@pytest.fixture(scope="session")
def engine():
    """The package under test; importing it loads libcogni_qmm.so (built on demand here)."""
    from cogni_ml_b200 import build as _build  # noqa: F401  (module without the .so dependency)
    import cogni_ml_b200
    return cogni_ml_b200


@pytest.fixture(scope="session")
def cuda(engine):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("this test is marked gpu and needs a CUDA device")
    return torch.device("cuda:0")
