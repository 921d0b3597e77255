"""Decode attention on the GPU through the C ABI against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from helpers_gpu import dev, pos_tensor, poisoned_cache

pytestmark = pytest.mark.gpu
AD, GQA = 256, 6
SCALE = 1.0 / 16.0


@pytest.fixture(autouse=True, params=[1, 2, 3, 4], ids=["mma", "tc", "ws", "wt"])
def decode_kernel(request, q27):
    """Every test of this module runs on every split-K kernel (warp-MMA, tcgen05, warp-specialised, warp-specialised with P V on tcgen05)."""
    q27.set_decode_kernel(request.param)
    yield request.param
    q27.set_decode_kernel(0)


def run_decode(q27, orc, T, nkvh, n, n_ctx=None, seed_shift=0, check=True, q8_1=False):
    from qwen27_engine_b200 import synth
    nqh = nkvh * GQA
    n_ctx = n_ctx or n + 11
    qn, qg, kf, vf = synth.decode_inputs(T, nqh, nkvh, n, start_kv=seed_shift)
    kc_ref, vc_ref = orc.fill_cache(kf, vf, n_ctx)
    kc = poisoned_cache(q27, kc_ref, nkvh, n_ctx, n)
    vc = poisoned_cache(q27, vc_ref, nkvh, n_ctx, n)
    o = torch.full((T, nqh, AD), float("nan"), device="cuda")
    q27.attn_decode(dev(qn), dev(qg), kc, vc, o, None, None, pos_tensor(n - T), T, SCALE, nqh, nkvh, n_ctx)
    torch.cuda.synchronize()
    out = o.cpu().numpy()
    if check:
        ref = orc.attn_ref(qn, qg, kc_ref, vc_ref, n - T, SCALE, nkvh, n_ctx)
        assert_close(out, ref, "decode T=%d nkvh=%d n=%d" % (T, nkvh, n))
    return out, (qn, qg, kc, vc, kc_ref, vc_ref)


def test_config1_cpu_checkable(q27, orc):
    """1 query token, 24 Q / 4 KV heads, KV length 1024."""
    run_decode(q27, orc, 1, 4, 1024)
    assert q27.device_status() == 0


@pytest.mark.parametrize("T", [1, 2, 3, 4])
@pytest.mark.parametrize("n", [4, 5, 7, 33, 63, 64, 65, 100, 127, 128, 129, 1000, 4096, 4100, 9472, 9473, 20011])
def test_decode_depths(q27, orc, T, n):
    if n < T:
        pytest.skip("fewer positions than query tokens")
    run_decode(q27, orc, T, 2, n)


@pytest.mark.parametrize("nkvh", [1, 2, 4])
def test_decode_head_counts(q27, orc, nkvh):
    run_decode(q27, orc, 4, nkvh, 3000)
    assert q27.device_status() == 0


def test_config2_spec_verify_32k(q27, orc):
    """4 query tokens (causal inside the block), 24 Q / 4 KV heads, q8_0 KV length 32,768."""
    run_decode(q27, orc, 4, 4, 32768)


def test_config3_long_context(q27, orc):
    for n in (30000, 100000, 150000):
        run_decode(q27, orc, 4, 4, n, n_ctx=n + 8)
    assert q27.device_status() == 0


def test_causal_inside_the_block(q27, orc):
    """Token t must not see the K/V of tokens t+1..: changing them leaves its output unchanged."""
    T, nkvh, n = 4, 1, 500
    out, (qn, qg, kc, vc, kc_ref, vc_ref) = run_decode(q27, orc, T, nkvh, n)
    kc2, vc2 = kc.clone(), vc.clone()
    n_ctx = n + 11
    # overwrite the last row (position n-1, visible to the last token only)
    kc2[: n_ctx * AD].view(n_ctx, AD)[n - 1] = 77
    vc2[: n_ctx * AD].view(n_ctx, AD)[n - 1] = 99
    o2 = torch.empty((T, nkvh * GQA, AD), device="cuda")
    q27.attn_decode(dev(qn), dev(qg), kc2, vc2, o2, None, None, pos_tensor(n - T), T, SCALE, nkvh * GQA, nkvh, n_ctx)
    torch.cuda.synchronize()
    o2 = o2.cpu().numpy()
    assert np.array_equal(o2[:3], out[:3]) and not np.array_equal(o2[3], out[3])


def test_run_twice_bitwise(q27, orc):
    a, _ = run_decode(q27, orc, 4, 4, 12345, check=False)
    b, _ = run_decode(q27, orc, 4, 4, 12345, check=False)
    assert np.array_equal(a, b)


def test_q8_1_epilogue(q27, orc):
    """With xq the result leaves as q8_1: exactly the oracle's q8_1 of the kernel's own f32 result."""
    T, nkvh, n = 4, 2, 2000
    nqh = nkvh * GQA
    out, (qn, qg, kc, vc, _, _) = run_decode(q27, orc, T, nkvh, n)
    xq = torch.zeros((T, nqh, AD), dtype=torch.int8, device="cuda")
    xd = torch.zeros((T * nqh * 8,), dtype=torch.float32, device="cuda")
    q27.attn_decode(dev(qn), dev(qg), kc, vc, None, xq, xd, pos_tensor(n - T), T, SCALE, nqh, nkvh, n + 11)
    torch.cuda.synchronize()
    rq, rd = orc.q8_1(out.reshape(-1))
    assert np.array_equal(xq.cpu().numpy().reshape(-1), rq) and np.array_equal(xd.cpu().numpy(), rd)


@pytest.mark.parametrize("n,cuts", [(1000, [0, 512, 1000]), (5000, [0, 1280, 2560, 3840, 5000]), (300, [0, 64, 300])])
def test_kv_length_partials_merge(q27, orc, n, cuts):
    """One sequence split by KV length (each slice a cache of its own, as on separate GPUs):
    per-slice partials + the log-sum-exp merge = the whole."""
    from qwen27_engine_b200 import synth
    T, nkvh = 4, 2
    nqh = nkvh * GQA
    qn, qg, kf, vf = synth.decode_inputs(T, nqh, nkvh, n)
    parts, refs = [], []
    full_k, full_v = orc.fill_cache(kf, vf, n)
    for lo, hi in zip(cuts, cuts[1:]):
        n_ctx = hi - lo + 3
        kc_ref, vc_ref = orc.fill_cache(kf[:, lo:hi], vf[:, lo:hi], n_ctx)
        kc = poisoned_cache(q27, kc_ref, nkvh, n_ctx, hi - lo)
        vc = poisoned_cache(q27, vc_ref, nkvh, n_ctx, hi - lo)
        part = torch.full((T, nqh, 258), float("nan"), device="cuda")
        q27.attn_decode_partial(dev(qn), kc, vc, part, pos_tensor(n - T), T, SCALE, nqh, nkvh, n_ctx, lo, hi - lo)
        parts.append(part)
        refs.append(orc.attn_partial(qn, full_k, full_v, n - T, SCALE, nkvh, n, lo, hi))
    allp = torch.stack(parts).contiguous()
    o = torch.empty((T, nqh, AD), device="cuda")
    q27.lse_merge(allp, len(parts), T * nqh * 258, T * nqh, dev(qg), o)
    torch.cuda.synchronize()
    whole = orc.attn_ref(qn, qg, full_k, full_v, n - T, SCALE, nkvh, n)
    assert_close(o.cpu().numpy(), whole, "merged slices")
    # each partial, normalised on its own, against the oracle's partial
    for part, ref in zip(parts, refs):
        a = part.cpu().numpy()
        live = ref[..., 1] > 0
        assert np.array_equal(a[..., 1] > 0, live)
        ya = a[..., 2:][live] / a[..., 1:2][live]
        yr = ref[..., 2:][live] / ref[..., 1:2][live]
        assert_close(ya, yr, "slice partial")
        lse_a = a[..., 0][live] + np.log(a[..., 1][live])
        lse_r = ref[..., 0][live] + np.log(ref[..., 1][live])
        assert np.abs(lse_a - lse_r).max() < 2e-3
    assert q27.device_status() == 0


def test_lse_merge_generic(q27, orc):
    rng = np.random.default_rng(5)
    nparts, rows = 7, 50
    parts = rng.standard_normal((nparts, rows, 258)).astype(np.float32)
    parts[..., 1] = np.abs(parts[..., 1]) + 0.1
    parts[3, :, 0] = -1e30   # an empty partial is neutral
    parts[3, :, 1:] = 0
    qg = rng.standard_normal((rows, 512)).astype(np.float32)
    ref = orc.lse_merge(parts, qg)
    o = torch.empty((rows, AD), device="cuda")
    q27.lse_merge(dev(parts), nparts, rows * 258, rows, dev(qg), o)
    torch.cuda.synchronize()
    assert np.abs(o.cpu().numpy() - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max())
    ref2 = orc.lse_merge(parts, None)
    q27.lse_merge(dev(parts), nparts, rows * 258, rows, None, o)
    torch.cuda.synchronize()
    assert np.abs(o.cpu().numpy() - ref2).max() <= 1e-5 * max(1.0, np.abs(ref2).max())


@pytest.mark.parametrize("T,nkvh,n", [(4, 2, 777), (1, 1, 5), (4, 4, 64), (3, 2, 129), (2, 1, 4100), (4, 4, 32768)])
def test_f16_kv_cache(q27, orc, T, nkvh, n):
    """The f16 KV cache variant of the decode kernel (config: the 32,768 spec-verify case also with f16 KV)."""
    from qwen27_engine_b200 import synth
    nqh = nkvh * GQA
    qn, qg, kf, vf = synth.decode_inputs(T, nqh, nkvh, n)
    kc_ref, vc_ref = orc.fill_cache(kf, vf, n + 5, q8=False)
    o = torch.empty((T, nqh, AD), device="cuda")
    try:
        q27.attn_decode(dev(qn), dev(qg), poisoned_cache(q27, kc_ref, nkvh, n + 5, n, False),
                        poisoned_cache(q27, vc_ref, nkvh, n + 5, n, False), o, None, None, pos_tensor(n - T), T, SCALE,
                        nqh, nkvh, n + 5, q8=False)
    except q27.Q27Error as e:
        assert e.code == q27.UNSUPPORTED
        pytest.skip("f16 KV decode not built: " + str(e))
    torch.cuda.synchronize()
    assert_close(o.cpu().numpy(), orc.attn_ref(qn, qg, kc_ref, vc_ref, n - T, SCALE, nkvh, n + 5, q8=False), "f16 KV")


@pytest.mark.parametrize("n,cuts", [(5000, [0, 2560, 5000]), (3000, [0, 1024, 2048, 3000])])
def test_kv_length_slices_exchanged_over_peer_memory(q27, orc, n, cuts):
    """The peer-memory exchange of the KV-length split, with all "ranks" emulated on one GPU one after
    the other (every wait finds its flag already set: kernels that wait on one another never run
    concurrently on one GPU): each rank pushes its slice into every rank's exchange buffer, each rank's
    waiting merge then gives the whole result, bit-identical to the gathered merge; three steps in a
    row exercise the step counter and the two parities of the buffers."""
    from qwen27_engine_b200 import synth
    T, nkvh = 4, 1
    nqh = nkvh * GQA
    nz = len(cuts) - 1
    rows = T * nqh
    bufs = [torch.zeros(q27.xbuf_bytes(nz, rows), dtype=torch.uint8, device="cuda") for _ in range(nz)]
    ptrs = [b.data_ptr() for b in bufs]
    for step in range(3):
        qn, qg, kf, vf = synth.decode_inputs(T, nqh, nkvh, n, start_kv=step)
        full_k, full_v = orc.fill_cache(kf, vf, n)
        slices = []
        for z in range(nz):
            lo, hi = cuts[z], cuts[z + 1]
            n_ctx = hi - lo + 3
            kc_ref, vc_ref = orc.fill_cache(kf[:, lo:hi], vf[:, lo:hi], n_ctx)
            slices.append((poisoned_cache(q27, kc_ref, nkvh, n_ctx, hi - lo), poisoned_cache(q27, vc_ref, nkvh, n_ctx, hi - lo),
                           n_ctx, lo, hi))
        parts = []
        for z, (kc, vc, n_ctx, lo, hi) in enumerate(slices):
            q27.attn_decode_partial_push(dev(qn), kc, vc, pos_tensor(n - T), T, SCALE, nqh, nkvh, n_ctx, lo, hi - lo, ptrs, z)
            part = torch.empty((T, nqh, 258), device="cuda")
            q27.attn_decode_partial(dev(qn), kc, vc, part, pos_tensor(n - T), T, SCALE, nqh, nkvh, n_ctx, lo, hi - lo)
            parts.append(part)
        gathered = torch.empty((T, nqh, AD), device="cuda")
        q27.lse_merge(torch.stack(parts).contiguous(), nz, rows * 258, rows, dev(qg), gathered)
        whole = orc.attn_ref(qn, qg, full_k, full_v, n - T, SCALE, nkvh, n)
        for z in range(nz):
            o = torch.full((T, nqh, AD), float("nan"), device="cuda")
            q27.lse_merge_wait(bufs[z], nz, rows, dev(qg), o)
            torch.cuda.synchronize()
            assert torch.equal(o, gathered), "rank %d, step %d" % (z, step)
            assert_close(o.cpu().numpy(), whole, "peer-memory merge, rank %d, step %d" % (z, step))
        assert int(bufs[0][:4].view(torch.int32).item()) == step + 1  # the step counter advanced
    assert q27.device_status() == 0


@pytest.mark.parametrize("n,cuts", [(5000, [0, 2560, 5000]), (3000, [0, 1024, 2048, 3000])])
def test_fused_exchange_equals_the_pair_of_calls(q27, orc, n, cuts):
    """q27b_attn_decode_exchange (one kernel pushes this rank's slice, waits for the others and writes the
    output) against the gathered merge. On one GPU the other ranks' slices are pushed first, with the push-only
    call, so that the rank under test finds them and never waits for a later launch; fresh buffers per rank
    under test (the other ranks' step counters do not advance here)."""
    from qwen27_engine_b200 import synth
    T, nkvh = 4, 1
    nqh = nkvh * GQA
    nz = len(cuts) - 1
    rows = T * nqh
    qn, qg, kf, vf = synth.decode_inputs(T, nqh, nkvh, n)
    slices, parts = [], []
    for z in range(nz):
        lo, hi = cuts[z], cuts[z + 1]
        n_ctx = hi - lo + 3
        kc_ref, vc_ref = orc.fill_cache(kf[:, lo:hi], vf[:, lo:hi], n_ctx)
        kc, vc = poisoned_cache(q27, kc_ref, nkvh, n_ctx, hi - lo), poisoned_cache(q27, vc_ref, nkvh, n_ctx, hi - lo)
        slices.append((kc, vc, n_ctx, lo, hi))
        part = torch.empty((T, nqh, 258), device="cuda")
        q27.attn_decode_partial(dev(qn), kc, vc, part, pos_tensor(n - T), T, SCALE, nqh, nkvh, n_ctx, lo, hi - lo)
        parts.append(part)
    gathered = torch.empty((T, nqh, AD), device="cuda")
    q27.lse_merge(torch.stack(parts).contiguous(), nz, rows * 258, rows, dev(qg), gathered)
    for me in range(nz):
        bufs = [torch.zeros(q27.xbuf_bytes(nz, rows), dtype=torch.uint8, device="cuda") for _ in range(nz)]
        ptrs = [b.data_ptr() for b in bufs]
        for z, (kc, vc, n_ctx, lo, hi) in enumerate(slices):
            if z != me:
                q27.attn_decode_partial_push(dev(qn), kc, vc, pos_tensor(n - T), T, SCALE, nqh, nkvh, n_ctx, lo, hi - lo, ptrs, z)
        torch.cuda.synchronize()
        kc, vc, n_ctx, lo, hi = slices[me]
        o = torch.full((T, nqh, AD), float("nan"), device="cuda")
        q27.attn_decode_exchange(dev(qn), dev(qg), kc, vc, o, pos_tensor(n - T), T, SCALE, nqh, nkvh, n_ctx, lo, hi - lo, ptrs, me)
        torch.cuda.synchronize()
        assert q27.device_status() == 0
        assert torch.equal(o, gathered), "rank %d" % me
        assert int(bufs[me][:4].view(torch.int32).item()) == 1  # its step counter advanced
        # and what it pushed is what the push-only call pushes
        other = (me + 1) % nz
        ref = [torch.zeros(q27.xbuf_bytes(nz, rows), dtype=torch.uint8, device="cuda") for _ in range(nz)]
        q27.attn_decode_partial_push(dev(qn), kc, vc, pos_tensor(n - T), T, SCALE, nqh, nkvh, n_ctx, lo, hi - lo,
                                     [b.data_ptr() for b in ref], me)
        torch.cuda.synchronize()
        per = rows * 258 * 8
        a0 = 256 + me * per
        assert torch.equal(bufs[other][a0:a0 + per], ref[other][a0:a0 + per])


def _tagged(parts, tag):
    """float rows -> the exchange buffer's words: {value, step tag} as int32 pairs."""
    w = torch.empty(parts.shape + (2,), dtype=torch.int32, device=parts.device)
    w[..., 0] = parts.contiguous().view(torch.int32)
    w[..., 1] = tag
    return w


def test_peer_memory_merge_reports_a_missing_slice(q27):
    """A slice that never arrives: the waiting merge gives up after its limit and says so in the status
    word (nothing hangs, nothing traps); the output is left alone."""
    nz, rows = 2, 6
    buf = torch.zeros(q27.xbuf_bytes(nz, rows), dtype=torch.uint8, device="cuda")
    words = buf[256:].view(torch.int32)[: 2 * nz * rows * 258 * 2].view(2, nz, rows, 258, 2)  # [parity][slice][row][word]
    parts = torch.randn((nz, rows, 258), device="cuda")
    parts[..., 1] = parts[..., 1].abs() + 0.5
    words[0, 0] = _tagged(parts[0], 1)  # slice 0 of step 1 is there, slice 1 is missing
    o = torch.full((rows, AD), 7.0, device="cuda")
    q27.lse_merge_wait(buf, nz, rows, None, o)
    assert q27.device_status() & 1
    assert bool((o == 7.0).all())
    # the buffer is out of step now (its CTAs left without the step's bookkeeping) and holds words of the
    # broken step: after a reset a complete step on the same buffer works again
    q27.xbuf_reset(buf)
    assert int(buf.max().item()) == 0
    words[0] = _tagged(parts, 1)  # parity 0 of step 1
    q27.lse_merge_wait(buf, nz, rows, None, o)
    want = torch.empty((rows, AD), device="cuda")
    q27.lse_merge(parts.contiguous(), nz, rows * 258, rows, None, want)
    torch.cuda.synchronize()
    assert q27.device_status() == 0
    assert torch.equal(o, want)
    assert int(buf[:4].view(torch.int32).item()) == 1  # the step counter advanced from zero
