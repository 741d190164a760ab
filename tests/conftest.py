"""pytest configuration: registers the ``gpu`` marker, puts the package
(``k100lc-kernels_b200/``), the oracle and the tests folder on ``sys.path``, and
provides the shared fixtures."""
from __future__ import annotations

import json
import pathlib
import sys

import numpy as np
import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
for p in (ROOT / "k100lc-kernels_b200", ROOT / "oracle", ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    """The committed reference vectors: (arrays, metadata)."""
    g = ROOT / "tests" / "golden"
    arrays = dict(np.load(g / "reference_vectors.npz"))
    meta = json.loads((g / "reference_vectors.json").read_text())["cases"]
    return arrays, meta


@pytest.fixture(scope="session")
def rt():
    """One engine per test session (the engine is process-global, like the
    reference's).  Fails loudly when the CUDA library or a device is missing."""
    from k100lc_kernels import Runtime
    return Runtime()
