"""Shared test set-up: import paths, the `gpu` marker, handles on the oracle and the library."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "orcasaq2-kernel_b200")
for p in (PKG, os.path.join(ROOT, "oracle"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


@pytest.fixture(scope="session")
def coracle():
    import exl3_ref
    return exl3_ref.COracle()


@pytest.fixture(scope="session")
def ext():
    """The ctypes binding of the CUDA library; GPU tests must go through it."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from orcasaq2 import _ext
    _ext.lib()          # raises if the library is missing: never fall back
    return _ext
