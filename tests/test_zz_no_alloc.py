"""q27b_attn_decode_noalloc: the decode entry point for callers that may not allocate device memory
(hosts with a device-memory budget fixed at start-up, hosts that drive several GPUs in lock step
and cannot afford the device-wide synchronisation of a cudaMalloc in the middle of a batch,
runtimes that own the allocator). Its split partials live in an array inside the library image.

The test calls it through the C ABI twice in a row, on two different problems, and compares each
result with the allocating entry point q27b_attn_decode on the same inputs: the two share their
kernels, so the outputs must agree to the tolerance of the path (they are in fact identical), and
the second call shows that what the first one left in the shared array does no harm.
A second test runs in a fresh process, where the no-allocation entry point is the first thing the
library is asked to do, and checks what the entry point exists for: the device's free memory is the
same before and after a call.
The file name makes pytest collect it last."""
import os
import subprocess
import sys
import numpy as np
import pytest
import torch

from conftest import assert_close
from helpers_gpu import dev, pos_tensor

pytestmark = pytest.mark.gpu
AD, GQA = 256, 6
SCALE = 1.0 / 16.0


def _case(q27, orc, T, nkvh, n, start):
    from qwen27_engine_b200 import synth
    nqh = nkvh * GQA
    n_ctx = n + 7
    qn, qg, kf, vf = synth.decode_inputs(T, nqh, nkvh, n, start_kv=start)
    kc, vc = orc.fill_cache(kf, vf, n_ctx)
    return dev(qn), dev(qg), dev(kc), dev(vc), nqh, n_ctx, (qn, qg, kc, vc)


def test_no_alloc_entry_point_matches_attn_decode_twice(q27, orc):
    # a long sequence first, then a short one with fewer query tokens: the second call finds the
    # first call's partials in the shared array
    for T, nkvh, n, start in ((4, 4, 9000, 0), (2, 4, 130, 1 << 22)):
        qn, qg, kc, vc, nqh, n_ctx, host = _case(q27, orc, T, nkvh, n, start)
        pos = pos_tensor(n - T)
        want = torch.empty((T, nqh, AD), device="cuda")
        q27.attn_decode(qn, qg, kc, vc, want, None, None, pos, T, SCALE, nqh, nkvh, n_ctx)
        got = torch.full((T, nqh, AD), float("nan"), device="cuda")
        q27.attn_decode_noalloc(qn, qg, kc, vc, got, None, None, pos, T, SCALE, nqh, nkvh, n_ctx)
        torch.cuda.synchronize()
        assert_close(got.cpu().numpy(), want.cpu().numpy(), "no-alloc vs attn_decode (T=%d n=%d)" % (T, n))
        assert np.array_equal(got.cpu().numpy(), want.cpu().numpy())
        # and both against the oracle, so that a shared mistake cannot hide
        ref = orc.attn_ref(host[0], host[1], host[2], host[3], n - T, SCALE, nkvh, n_ctx)
        assert_close(got.cpu().numpy(), ref, "no-alloc vs oracle")
    assert q27.device_status() == 0


def test_no_alloc_entry_point_rejects_what_does_not_fit(q27):
    # 161 KV heads need at least 161 chunk partials, one more than the array holds, on any GPU
    nkvh = 161
    nqh = nkvh * GQA
    qn = torch.zeros((1, nqh, AD), device="cuda")
    qg = torch.zeros((1, nqh, 512), device="cuda")
    cache = torch.zeros(q27.kv_cache_bytes(nkvh, 64), dtype=torch.uint8, device="cuda")
    o = torch.zeros((1, nqh, AD), device="cuda")
    with pytest.raises(q27.Q27Error) as e:
        q27.attn_decode_noalloc(qn, qg, cache, cache, o, None, None, pos_tensor(0), 1, SCALE, nqh, nkvh, 64)
    assert e.value.code == q27.BAD_SHAPE and "160" in str(e.value)


_FRESH = r"""
import sys
sys.path.insert(0, %(root)r)
sys.path.insert(0, %(tests)r)
import numpy as np, torch
import __graft_entry__ as ge
import oracle
q = ge.load_package()
from qwen27_engine_b200 import synth
T, nkvh, n = 4, 4, 5000
nqh, n_ctx = nkvh * 6, n + 7
qn, qg, kf, vf = synth.decode_inputs(T, nqh, nkvh, n)
kc, vc = oracle.fill_cache(kf, vf, n_ctx)
d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
dq, dg, dk, dv = d(qn), d(qg), d(kc), d(vc)
pos = torch.tensor([n - T], dtype=torch.int32, device="cuda")
o = torch.full((T, nqh, 256), float("nan"), device="cuda")
torch.cuda.synchronize()
# first call of the library in this process: looks up the array and loads the kernels
q.attn_decode_noalloc(dq, dg, dk, dv, o, None, None, pos, T, 1.0 / 16.0, nqh, nkvh, n_ctx)
torch.cuda.synchronize()
free0 = torch.cuda.mem_get_info()[0]
o2 = torch.full((T, nqh, 256), float("nan"), device="cuda")  # (allocated before the measured call)
torch.cuda.synchronize()
free1 = torch.cuda.mem_get_info()[0]
q.attn_decode_noalloc(dq, dg, dk, dv, o2, None, None, pos, T, 1.0 / 16.0, nqh, nkvh, n_ctx)
torch.cuda.synchronize()
free2 = torch.cuda.mem_get_info()[0]
ref = oracle.attn_ref(qn, qg, kc, vc, n - T, 1.0 / 16.0, nkvh, n_ctx)
err = float(np.abs(o.cpu().numpy() - ref).max()); rms = float(np.sqrt((ref ** 2).mean()))
print("RESULT", free1 - free2, err, rms, int(torch.equal(o, o2)), q.device_status(), q.workspace_query())
"""


def test_no_alloc_entry_point_in_a_fresh_process_leaves_free_memory_alone():
    """Fresh process, q27b_attn_decode_noalloc before any other entry point: correct against the oracle,
    and across its second call (the first one loads the kernels, which CUDA does lazily and which takes
    device memory whoever launches them) cudaMemGetInfo reports the same free bytes; the library's own
    workspace was never allocated."""
    code = _FRESH % {"root": os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                     "tests": os.path.dirname(os.path.abspath(__file__))}
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT")][0]
    parts = line.split(None, 6)
    used, err, rms, same, status = int(parts[1]), float(parts[2]), float(parts[3]), int(parts[4]), int(parts[5])
    assert used == 0, "free device memory changed by %d bytes across a no-alloc call" % used
    assert err <= 2e-3 and err <= 1e-2 * rms and same == 1 and status == 0
    assert parts[6].startswith("(0, 0, 0, False)"), "the allocating workspace was touched: " + parts[6]
