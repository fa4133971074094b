import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def ref():
    """The reference's own headers compiled by oracle/build_oracle.py."""
    from oracle import build_oracle, refapi
    build_oracle.build_reference()
    if not refapi.have_reference():
        pytest.skip("oracle/_ref/libsdca_ref.so is not built and the reference tree is absent")
    return refapi.reference()


@pytest.fixture(scope="session")
def ref_accurate():
    """The reference compiled with SDCA_ACCURATE_MATH (exact recomputation of t)."""
    from oracle import build_oracle, refapi
    build_oracle.build_reference()
    if not os.path.exists(refapi.ReferenceAccurate.path):
        pytest.skip("oracle/_ref/libsdca_ref_accurate.so is not built and the reference tree is absent")
    return refapi.reference_accurate()


@pytest.fixture(scope="session")
def hostsim():
    from tests.hostsim import build as hb
    return hb.load()


@pytest.fixture(scope="session")
def cuda_lib():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import libsdca_b200
    libsdca_b200.lib()  # raises if the library is not built: no fallback
    return libsdca_b200
