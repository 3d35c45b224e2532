"""Shared fixtures.  Tests marked ``gpu`` need a B200 and call the CUDA library through its C ABI;
everything else runs on the CPU (oracle checks, host logic, ABI surface)."""

from __future__ import annotations

import os
import sys

import numpy as np
import pytest

# The library reads its tuning knobs (YULE_GEMM_*, YULE_TP_*, YULE_CUDA_*) only in a process started with this
# switch; some tests select a kernel route through them.
os.environ.setdefault("YULE_CUDA_DEBUG", "1")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def native_libs():
    """Build (if stale) the package's libraries and the oracle once per session."""
    from yule_b200 import build
    from oracle import build_oracle
    build.build_synth()
    build.build_cuda()
    build_oracle.build_oracle()
    build_oracle.build_ref()
    build_oracle.build_ref_cuda()
    return True


@pytest.fixture(scope="session")
def oracle(native_libs):
    from oracle import oracle as o
    return o


@pytest.fixture(scope="session")
def backend(native_libs):
    """One CUDA context for the whole session; fails loudly when the library or device is missing."""
    from yule_b200 import CudaB200Backend
    b = CudaB200Backend(0)
    yield b
    b.close()


def guarded_rel_err(y: np.ndarray, ref: np.ndarray) -> float:
    """max_i |y - ref| / max(|ref_i|, 1e-3 * max|ref|): relative error with a floor, so that entries
    near zero are judged against the vector's scale instead of against themselves."""
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    floor = 1e-3 * max(np.abs(ref).max(), 1e-30)
    return float((np.abs(y - ref) / np.maximum(np.abs(ref), floor)).max())


# Tolerance of every matvec / attention / logits comparison: max relative error 1e-3 with fp32
# accumulation on both sides (the floor above makes it well posed near zero).
REL_TOL = 1e-3
