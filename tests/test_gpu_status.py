"""The failure path without a failure of the GPU: a bounded wait that runs out is reported through
the device status word, nothing hangs or traps, and the library keeps working afterwards."""
import time

import pytest

from test_gpu_decode import run_decode

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_the_context_stays_usable(q27, orc):
    assert q27.device_status() == 0
    t0 = time.time()
    q27.debug_expire_wait()          # one warp waits on a barrier that nobody arrives at
    st = q27.device_status()         # synchronises: the wait gives up after its limit
    dt = time.time() - t0
    assert st & 1, "ST_WAIT_EXPIRED must be set"
    assert 1.0 < dt < 30.0, "the limit is about two seconds (took %.1f s)" % dt
    assert q27.device_status() == 0  # reading the status cleared it
    run_decode(q27, orc, T=4, nkvh=1, n=700)  # same context, correct results
    assert q27.device_status() == 0
