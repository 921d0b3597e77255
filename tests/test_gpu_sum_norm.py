"""x += sum of the ranks' partial rows, RMSNorm, q8_1 (the step after the attention output
projection, the reference's sum_norm_q8): one GPU, and the peer-memory exchange with the ranks of a
group run one after the other on this GPU (every push before any wait, so nothing waits for a later
launch)."""
import numpy as np
import pytest
import torch

from helpers_gpu import dev

pytestmark = pytest.mark.gpu
EPS = 1e-6


def inputs(rows, n, world, step=0):
    from qwen27_engine_b200 import synth
    x = synth.normal(synth.SEED_Q, (rows, n), start=step << 20)
    w = 1.0 + 0.1 * synth.normal(synth.SEED_GATE, (n,))
    parts = [0.3 * synth.normal(synth.SEED_K, (rows, n), start=(step * 8 + r) << 22) for r in range(world)]
    return x, w.astype(np.float32), parts


def check(orc, x_gpu, h_gpu, xq, xd, x, parts, w):
    xn, h = orc.sum_norm(x, parts, w, EPS)
    assert np.array_equal(x_gpu, xn)                       # f32 adds in the same order: exact
    np.testing.assert_allclose(h_gpu, h, rtol=2e-6, atol=1e-7)
    rq, rd = orc.q8_1(h_gpu.reshape(-1))                   # q8_1 of the kernel's own f32 result: exact
    assert np.array_equal(xq.reshape(-1), rq) and np.array_equal(xd, rd)


@pytest.mark.parametrize("rows,n", [(1, 5120), (4, 5120), (37, 5120), (3, 96), (2, 16384), (5, 1056)])
def test_sum_norm_q8_one_gpu(q27, orc, rows, n):
    x, w, parts = inputs(rows, n, 1)
    dx = dev(x)
    h = torch.full((rows, n), float("nan"), device="cuda")
    xq = torch.zeros((rows, n), dtype=torch.int8, device="cuda")
    xd = torch.zeros((rows * n // 32,), dtype=torch.float32, device="cuda")
    q27.sum_norm_q8(dx, dev(parts[0]), n, rows, dev(w), EPS, h, xq, xd)
    torch.cuda.synchronize()
    check(orc, dx.cpu().numpy(), h.cpu().numpy(), xq.cpu().numpy(), xd.cpu().numpy(), x, parts, w)
    # without h
    dx2 = dev(x)
    xq2 = torch.zeros_like(xq)
    xd2 = torch.zeros_like(xd)
    q27.sum_norm_q8(dx2, dev(parts[0]), n, rows, dev(w), EPS, None, xq2, xd2)
    torch.cuda.synchronize()
    assert torch.equal(xq2, xq) and torch.equal(xd2, xd) and torch.equal(dx2, dx)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sum_norm_q8_exchanged_over_peer_memory(q27, orc, world):
    rows, n = 4, 5120
    bufs = [q27.xbuf_alloc_bytes(q27.sum_xbuf_bytes(world, rows, n)) for _ in range(world)]
    try:
        for step in range(3):                               # both parities of the data area, the epoch advancing
            x, w, parts = inputs(rows, n, world, step)
            for r in range(world):
                q27.sum_push(dev(parts[r]), n, rows, r, bufs)
            outs = []
            for r in range(world):
                dx = dev(x)
                h = torch.full((rows, n), float("nan"), device="cuda")
                xq = torch.zeros((rows, n), dtype=torch.int8, device="cuda")
                xd = torch.zeros((rows * n // 32,), dtype=torch.float32, device="cuda")
                q27.sum_norm_q8_wait(dx, bufs[r], world, n, rows, dev(w), EPS, h, xq, xd)
                outs.append((dx, h, xq, xd))
            torch.cuda.synchronize()
            assert q27.device_status() == 0
            for dx, h, xq, xd in outs:
                check(orc, dx.cpu().numpy(), h.cpu().numpy(), xq.cpu().numpy(), xd.cpu().numpy(), x, parts, w)
            for dx, h, xq, xd in outs[1:]:                  # every rank holds the same bits
                assert torch.equal(dx, outs[0][0]) and torch.equal(h, outs[0][1]) and torch.equal(xq, outs[0][2])
    finally:
        for b in bufs:
            q27.xbuf_free(b)


@pytest.mark.parametrize("world", [2, 4])
def test_fused_exchange_equals_push_and_wait(q27, orc, world):
    """q27b_sum_exchange_norm_q8 (one kernel pushes this rank's rows, waits for the others and normalises) against
    the pair of calls. On one GPU the other ranks push first (push-only call), so that the rank under test never
    waits for a later launch; fresh buffers per rank under test."""
    rows, n = 4, 5120
    x, w, parts = inputs(rows, n, world, 1)

    def run(me, fused):
        bufs = [q27.xbuf_alloc_bytes(q27.sum_xbuf_bytes(world, rows, n)) for _ in range(world)]
        try:
            for r in range(world):
                if r != me or not fused:
                    q27.sum_push(dev(parts[r]), n, rows, r, bufs)
            dx = dev(x)
            h = torch.full((rows, n), float("nan"), device="cuda")
            xq = torch.zeros((rows, n), dtype=torch.int8, device="cuda")
            xd = torch.zeros((rows * n // 32,), dtype=torch.float32, device="cuda")
            if fused:
                q27.sum_exchange_norm_q8(dx, dev(parts[me]), n, rows, me, bufs, dev(w), EPS, h, xq, xd)
            else:
                q27.sum_norm_q8_wait(dx, bufs[me], world, n, rows, dev(w), EPS, h, xq, xd)
            torch.cuda.synchronize()
            assert q27.device_status() == 0
            return dx, h, xq, xd
        finally:
            for b in bufs:
                q27.xbuf_free(b)

    for me in range(world):
        a, b = run(me, True), run(me, False)
        for u, v in zip(a, b):
            assert torch.equal(u, v), "rank %d" % me


def test_sum_norm_wait_reports_a_missing_rank(q27):
    """Rank 1 never pushes: rank 0's wait runs out (about a second), the status word says so, the
    context stays usable."""
    rows, n, world = 2, 5120, 2
    bufs = [q27.xbuf_alloc_bytes(q27.sum_xbuf_bytes(world, rows, n)) for _ in range(world)]
    try:
        x, w, parts = inputs(rows, n, world)
        q27.sum_push(dev(parts[0]), n, rows, 0, bufs)
        dx = dev(x)
        q27.sum_norm_q8_wait(dx, bufs[0], world, n, rows, dev(w), EPS, None, None, None)
        torch.cuda.synchronize()
        assert q27.device_status() == 1  # ST_WAIT_EXPIRED
        assert q27.device_status() == 0
    finally:
        for b in bufs:
            q27.xbuf_free(b)


def test_sum_norm_q8_against_the_reference_kernel_fixture(q27):
    """The library's kernel against the outputs of the reference's own sum_norm_q8 kernel (B200 fixture)."""
    import os
    from conftest import ROOT
    from golden_cases import SUM_NORM_EPS, sum_norm_inputs
    g = np.load(os.path.join(ROOT, "tests", "golden", "ref_sum_norm_b200.npz"))
    x, part, w = sum_norm_inputs()
    rows, n = x.shape
    dx = dev(x)
    h = torch.empty((rows, n), device="cuda")
    xq = torch.zeros((rows, n), dtype=torch.int8, device="cuda")
    xd = torch.zeros((rows * n // 32,), dtype=torch.float32, device="cuda")
    q27.sum_norm_q8(dx, dev(part), n, rows, dev(w), SUM_NORM_EPS, h, xq, xd)
    torch.cuda.synchronize()
    assert np.array_equal(dx.cpu().numpy(), g["x"])
    np.testing.assert_allclose(h.cpu().numpy(), g["h"], rtol=2e-6, atol=1e-7)
    off = xq.cpu().numpy().astype(np.int32) - g["xq"].astype(np.int32)
    assert np.abs(off).max() <= 1 and (off != 0).mean() <= 1e-3
    np.testing.assert_allclose(xd.cpu().numpy(), g["xd"], rtol=1e-3)
