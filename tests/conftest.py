"""pytest configuration: the `gpu` marker, and shared fixtures (golden vectors, oracles)."""

import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Outputs of the reference itself on seeded inputs (tests/golden/make_golden.py)."""
    return np.load(REPO / "tests" / "golden" / "reference_cpu.npz")


@pytest.fixture(scope="session")
def golden_extra():
    """Second fixture file of the same generator: casts over every dtype pair, comparisons with NaN and
    signed zeros, pow with other exponents, min/max over NaN / signed-zero slices, non-finite matmul."""
    return np.load(REPO / "tests" / "golden" / "reference_cpu_extra.npz")


@pytest.fixture(scope="session")
def port():
    from oracle.oracle import PortOracle

    return PortOracle()


@pytest.fixture(scope="session")
def nt():
    """The product package; on a GPU box every op runs through libnt_b200.so."""
    import nanotorch_b200

    # the parity tests use small and ragged shapes on purpose: send every fp32 product of modes 1 and 3 to
    # the tensor-core kernel, not only those above the library's default size threshold
    nanotorch_b200._C.set_matmul_tc_min_macs(0)
    return nanotorch_b200
