import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    def load(name):
        with np.load(GOLDEN / f"{name}.npz") as data:
            return {k: data[k] for k in data.files}

    return load


@pytest.fixture(scope="session", autouse=True)
def _built_checkers():
    """Make sure the C oracle exists before any test touches it."""
    from oracle.build_oracle import build_c_oracle

    build_c_oracle()
