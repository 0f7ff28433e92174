import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def pkg():
    return entry.load_package()


@pytest.fixture(scope="session")
def synth(pkg):
    return pkg.synth


@pytest.fixture(scope="session")
def ops():
    """The ctypes binding; building is attempted once if the library is missing."""
    lib = os.path.join(entry.PKG_DIR, "libb200attn.so")
    if not os.path.exists(lib):
        entry.build()
    return entry.load_ops()


@pytest.fixture(scope="session")
def oracle():
    from oracle import cpu_oracle
    cpu_oracle.build()
    return cpu_oracle


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


def allclose_report(got, want, atol, rtol):
    import numpy as np
    err = np.abs(got - want)
    bound = atol + rtol * np.abs(want)
    bad = err > bound
    return (not bad.any()), f"max abs err {err.max():.3e}, worst excess {(err - bound).max():.3e}, {int(bad.sum())} of {bad.size} outside"
