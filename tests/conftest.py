"""pytest configuration: markers, import paths, shared fixtures."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = ROOT / "tests" / "golden"
for path in (str(ROOT), str(GOLDEN)):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (runs on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir() -> Path:
    return GOLDEN


@pytest.fixture(scope="session")
def golden_exact():
    return np.load(GOLDEN / "exact_reference_outputs.npz")


@pytest.fixture(scope="session")
def golden_paged():
    return np.load(GOLDEN / "paged_reference_outputs.npz")


@pytest.fixture(scope="session")
def golden_seed():
    return np.load(GOLDEN / "seed_reference_outputs.npz")
