"""Shared test plumbing: the `gpu` marker, the repo root on sys.path, seeded input builders."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); deselected on CPU-only machines with -m 'not gpu'")


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(ROOT / "tests" / "golden" / "golden.npz")


@pytest.fixture(scope="session")
def golden_rope():
    import numpy as np

    return np.load(ROOT / "tests" / "golden" / "golden_rope.npz")
