import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def zo():
    import oracle
    return oracle.Oracle()


@pytest.fixture(scope="session")
def zr():
    import oracle
    if not oracle.reference_available():
        try:
            oracle.build(with_reference=True)
        except Exception:
            pass
    if not oracle.reference_available():
        pytest.skip("compiled reference (oracle/_ref/libzenref.so) not present")
    return oracle.Reference()


def lcg_bytes(seed: int, n: int) -> np.ndarray:
    """The byte stream the reference's fixtures draw from: state = state*1664525 + 1013904223 (mod 2^32), top byte."""
    out = np.empty(n, np.uint8)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = s >> 24
    return out


def max_abs_over_max_ref(got, ref) -> float:
    """The reference's own GPU parity metric (tools/hip_parity.cpp:126-134): max|got-ref| / max|ref|."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    mr = np.abs(ref).max()
    ma = np.abs(got - ref).max()
    return float(ma / mr) if mr > 0 else float(ma)
