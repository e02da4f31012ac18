"""pytest configuration: the `gpu` marker and import paths."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def xp_gpu():
    """The CUDA path as a namespace; fails (never skips) when the library is missing."""
    import cumo_b200

    return cumo_b200
