"""Test configuration: markers, import paths, and the fixture loader."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
for p in (str(ROOT), str(GOLDEN)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / f"{name}.npz") as z:
        return {k: z[k] for k in z.files}


@pytest.fixture(scope="session")
def golden():
    return load_golden


@pytest.fixture(autouse=True)
def _kernel_status_stays_clear(request):
    """After every GPU test: no kernel gave up on a bounded wait (the status words of the library are 0)."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    from echokv_b200 import _native as N
    assert N.lib.echokv_kernel_status(1) == 0
