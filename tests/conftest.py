import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the B200 box)")


@pytest.fixture(scope="session")
def orc():
    """The CPU checker (oracle/), built on demand."""
    from oracle import oracle

    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def cm():
    """The product package; importing it loads the C-ABI library."""
    import camelid_b200

    return camelid_b200
