"""pytest configuration: the `gpu` marker and shared fixtures."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with `-m gpu`")


@pytest.fixture(scope="session")
def golden():
    """name -> dict of numpy arrays for every fixture file in tests/golden/."""
    return {p.stem: dict(np.load(p, allow_pickle=False)) for p in sorted(GOLDEN.glob("*.npz"))}
