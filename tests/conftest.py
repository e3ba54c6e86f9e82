"""Shared test plumbing: markers, import paths, golden fixtures and the CPU oracle."""
import hashlib
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")
for path in (ROOT, GOLDEN):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def sha(array) -> str:
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()[:32]


@pytest.fixture(scope="session")
def golden():
    with open(os.path.join(GOLDEN, "codec.json")) as handle:
        return json.load(handle)


@pytest.fixture(scope="session")
def golden_tables():
    return np.load(os.path.join(GOLDEN, "tables.npz"))


@pytest.fixture(scope="session")
def oracle():
    """The C oracle, compiled on first use (test infrastructure only)."""
    from oracle import lct_oracle

    lct_oracle.build()
    return lct_oracle
