from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    with np.load(ROOT / "tests" / "golden" / "golden.npz") as data:
        return {name: data[name] for name in data.files}


@pytest.fixture(scope="session")
def oracle():
    import oracle as module

    module.build(ref=True)
    return module
