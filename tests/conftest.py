"""pytest configuration.

``-m "not gpu"`` runs the oracle/golden checks, the host logic and the C-ABI symbol
checks on a CPU-only machine.  ``-m gpu`` runs the parity tests proper: every one calls
the CUDA kernels through the C ABI and compares with the CPU oracle on the same seeded
inputs.  GPU tests are skipped (not passed) when no CUDA device is present.
"""
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def fg():
    import flaggems_b200

    return flaggems_b200


@pytest.fixture(autouse=True)
def _device_healthy(request):
    """After every GPU test, a kernel whose bounded wait gave up must not go unnoticed."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        from flaggems_b200 import _lib

        torch.cuda.synchronize()
        assert _lib.device_status(reset=True) == 0, "a kernel reported a timed-out wait"
