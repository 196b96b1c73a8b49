import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (checker only)."""
    from oracle import oracle

    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def backend():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import magnitude_b200 as mb

    be = mb.Backend(0)
    yield be
    be.close()
