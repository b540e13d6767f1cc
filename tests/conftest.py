"""Shared fixtures.  ``gpu`` marks tests that need a CUDA device (B200)."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device; run on the B200 box with -m gpu")


@pytest.fixture(scope="session")
def golden():
    return np.load(ROOT / "tests" / "golden" / "reference_vectors.npz")


@pytest.fixture(scope="session")
def oracle():
    from oracle import nq_oracle

    nq_oracle.build()
    return nq_oracle
