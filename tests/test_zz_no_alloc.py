"""q27b_attn_decode_noalloc: the decode entry point for callers that may not allocate device memory
(hosts with a device-memory budget fixed at start-up, hosts that drive several GPUs in lock step
and cannot afford the device-wide synchronisation of a cudaMalloc in the middle of a batch,
runtimes that own the allocator). Its split partials live in an array inside the library image.

The test calls it through the C ABI twice in a row, on two different problems, and compares each
result with the allocating entry point q27b_attn_decode on the same inputs: the two share their
kernels, so the outputs must agree to the tolerance of the path (they are in fact identical), and
the second call shows that what the first one left in the shared array does no harm.
The file name makes pytest collect it last."""
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
