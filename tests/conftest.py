"""Shared test helpers. GPU tests are marked `gpu` and call the library through its C ABI
(ctypes); everything else runs on CPU only."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Tolerance of the path on floating outputs: max |a - b| <= 2e-3 and <= 1e-2 of the reference RMS.
ABS_TOL = 2e-3
REL_TOL = 1e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def q27():
    import __graft_entry__ as ge
    lib = os.path.join(ge.PKG_DIR, "libq27b_attn.so")
    if not os.path.exists(lib):
        ge.build()
    return ge.load_package()


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.lib()
    return oracle


def err_stats(a, ref):
    a = np.asarray(a, np.float64)
    ref = np.asarray(ref, np.float64)
    d = np.abs(a - ref)
    rms = float(np.sqrt((ref ** 2).mean()))
    return float(d.max()), rms, float(np.sqrt((d ** 2).sum()) / max(np.sqrt((ref ** 2).sum()), 1e-30))


def assert_close(a, ref, what="", abs_tol=ABS_TOL, rel_tol=REL_TOL):
    finite = bool(np.isfinite(np.asarray(a)).all())
    assert finite, "%s: non-finite values" % what
    mx, rms, l2 = err_stats(a, ref)
    assert mx <= abs_tol and mx <= rel_tol * rms and l2 <= rel_tol, \
        "%s: max err %.3e, ref rms %.3e, rel L2 %.3e" % (what, mx, rms, l2)
    return mx, rms, l2
