"""pytest configuration: the `gpu` marker, import paths and shared fixtures."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
for p in (REPO, REPO / "torch-webgpu_b200", REPO / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Inputs and PyTorch CPU ATen outputs committed under tests/golden/."""
    with np.load(REPO / "tests" / "golden" / "aten_golden.npz") as z:
        return {k: z[k] for k in z.files}
