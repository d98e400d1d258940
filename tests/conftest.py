"""Shared test set-up: the `gpu` marker, import paths, and the device fixture the ported reference tests take."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "tensix-kernels_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def device():
    """The one device of the session, as the reference's conftest.py:14-19 provides it."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from common import ttnn_like as ttnn

    d = ttnn.open_device(device_id=0)
    yield d
    ttnn.close_device(d)
