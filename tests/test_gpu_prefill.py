"""Prefill attention (int8 Q K^T on tcgen05) on the GPU through the C ABI against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from conftest import assert_close
from helpers_gpu import dev, pos_tensor, poisoned_cache

pytestmark = pytest.mark.gpu
AD, GQA = 256, 6
SCALE = 1.0 / 16.0


def make_case(orc, M, pos0, nkvh, n_ctx=None):
    from qwen27_engine_b200 import synth
    nqh = nkvh * GQA
    n = pos0 + M
    n_ctx = n_ctx or n + 9
    qn = synth.normal(synth.SEED_Q, (M, nqh, AD))
    qg = np.zeros((M, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (M, nqh, AD))
    kf = synth.normal(synth.SEED_K, (nkvh, n, AD))
    vf = synth.normal(synth.SEED_V, (nkvh, n, AD))
    kc, vc = orc.fill_cache(kf, vf, n_ctx)
    return qn, qg, kc, vc, n, n_ctx


@pytest.mark.parametrize("rows,npos,p0", [(128, 64, 0), (37, 64, 100), (128, 17, 5), (1, 1, 63)])
def test_integer_stage_bit_exact(q27, orc, rows, npos, p0):
    """int8 Q bytes, f32 Q scales and the per-32-block int32 Q K^T accumulators: bit-exact."""
    from qwen27_engine_b200 import synth
    nkvh, kh, n_ctx = 2, 1, 300
    x = synth.normal(synth.SEED_Q, (rows, AD), start=12345)
    x[0, :32] = 0
    kf = synth.normal(synth.SEED_K, (nkvh, n_ctx, AD))
    kc, _ = orc.fill_cache(kf, kf, n_ctx)
    q_i8 = torch.zeros((rows, AD), dtype=torch.int8, device="cuda")
    q_sc = torch.zeros((rows, 8), dtype=torch.float32, device="cuda")
    acc = torch.zeros((rows, npos, 8), dtype=torch.int32, device="cuda")
    q27.prefill_qk_debug(dev(x), rows, SCALE, dev(kc), nkvh, n_ctx, kh, p0, npos, q_i8, q_sc, acc)
    torch.cuda.synchronize()
    rq, rd = orc.quant_q_i8(x, SCALE)
    assert np.array_equal(q_i8.cpu().numpy(), rq)
    assert np.array_equal(q_sc.cpu().numpy(), rd)
    kq = kc[: nkvh * n_ctx * AD].view(np.int8).reshape(nkvh, n_ctx, AD)[kh, p0:p0 + npos]
    assert np.array_equal(acc.cpu().numpy(), orc.qk_i32(rq, kq))
    assert q27.device_status() == 0


# {pos0, M} of the reference's own check (tools/bench_attn.cu:77), at sizes the oracle finishes quickly
@pytest.mark.parametrize("pos0,M", [(0, 37), (0, 128), (1000, 64), (5000, 128), (0, 1), (63, 2), (300, 200), (129, 257)])
@pytest.mark.parametrize("nkvh", [1, 2])
def test_prefill_matches_oracle(q27, orc, pos0, M, nkvh):
    if nkvh == 2 and M > 130:
        pytest.skip("covered with one KV head")
    qn, qg, kc_ref, vc_ref, n, n_ctx = make_case(orc, M, pos0, nkvh)
    nqh = nkvh * GQA
    o = torch.full((M, nqh, AD), float("nan"), device="cuda")
    q27.attn_prefill(dev(qn), dev(qg), poisoned_cache(q27, kc_ref, nkvh, n_ctx, n),
                     poisoned_cache(q27, vc_ref, nkvh, n_ctx, n), o, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx)
    torch.cuda.synchronize()
    ref = orc.attn_prefill_i8(qn, qg, kc_ref, vc_ref, pos0, SCALE, nkvh, n_ctx)
    assert_close(o.cpu().numpy(), ref, "prefill pos0=%d M=%d" % (pos0, M))
    assert q27.device_status() == 0


@pytest.mark.parametrize("depth_hint", [8000, -1])
def test_prefill_split_kv(q27, orc, depth_hint):
    """With a depth hint the positions are split over CTAs and merged by log-sum-exp."""
    pos0, M, nkvh = 8000, 70, 1
    qn, qg, kc_ref, vc_ref, n, n_ctx = make_case(orc, M, pos0, nkvh)
    o = torch.full((M, 6, AD), float("nan"), device="cuda")
    q27.attn_prefill(dev(qn), dev(qg), dev(kc_ref), dev(vc_ref), o, pos_tensor(pos0), M, SCALE, 6, nkvh, n_ctx,
                     depth_hint=depth_hint)
    torch.cuda.synchronize()
    ref = orc.attn_prefill_i8(qn, qg, kc_ref, vc_ref, pos0, SCALE, nkvh, n_ctx)
    assert_close(o.cpu().numpy(), ref, "prefill split hint=%d" % depth_hint)


def test_prefill_chunk_2048_rows_sampled(q27, orc):
    """Config: 2048 new tokens on a 32,768-token prefix, 24 Q / 4 KV heads. The oracle checks the
    first, a middle and the last 4 tokens of the chunk (all heads)."""
    pos0, M, nkvh = 32768, 2048, 4
    qn, qg, kc_ref, vc_ref, n, n_ctx = make_case(orc, M, pos0, nkvh, n_ctx=pos0 + M)
    nqh = nkvh * GQA
    o = torch.full((M, nqh, AD), float("nan"), device="cuda")
    q27.attn_prefill(dev(qn), dev(qg), dev(kc_ref), dev(vc_ref), o, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx,
                     depth_hint=pos0)
    torch.cuda.synchronize()
    out = o.cpu().numpy()
    assert np.isfinite(out).all()
    for lo in (0, 1022, 2044):
        ref = orc.attn_prefill_i8(qn, qg, kc_ref, vc_ref, pos0, SCALE, nkvh, n_ctx, lo, lo + 4)
        assert_close(out[lo:lo + 4], ref[lo:lo + 4], "tokens %d..%d" % (lo, lo + 3))
    assert q27.device_status() == 0


_cfg4 = {}


def _config4_case(orc, pos0):
    """The prefill configuration of the metric (M = 2048, 24 Q / 4 KV heads) on a prefix of pos0 tokens;
    built once per prefix (150,048 positions x 4 heads of N(0,1) rows take a while on the host)."""
    if pos0 not in _cfg4:
        _cfg4.clear()  # one prefix at a time: a case is 1.2 GB of host memory
        _cfg4[pos0] = make_case(orc, 2048, pos0, 4, n_ctx=pos0 + 2048)
    return _cfg4[pos0]


@pytest.mark.parametrize("kernel", [1, 2], ids=["int8", "f16qk"])
@pytest.mark.parametrize("pos0", [0, 148000])
def test_prefill_config4_at_both_ends(q27, orc, pos0, kernel):
    """The metric's prefill chunk at the two depths that the 32,768 test above leaves out: no prefix at
    all (causal only, tiles of 1..16 K/V tiles) and 148,000 tokens (the depth the TOPS figure is quoted
    at, where the tail split cuts the first query tiles into 5 pieces). Both kernels; the oracle checks
    token ranges at the start, around tile and split boundaries, and at the end."""
    M, nkvh = 2048, 4
    nqh = nkvh * GQA
    qn, qg, kc_ref, vc_ref, n, n_ctx = _config4_case(orc, pos0)
    o = torch.full((M, nqh, AD), float("nan"), device="cuda")
    q27.set_prefill_kernel(kernel)
    try:
        q27.attn_prefill(dev(qn), dev(qg), dev(kc_ref), dev(vc_ref), o, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx,
                         True, pos0)
        torch.cuda.synchronize()
    finally:
        q27.set_prefill_kernel(0)
    out = o.cpu().numpy()
    assert np.isfinite(out).all()
    for lo in (0, 126, 510, 1022, 2044):
        if kernel == 1:
            ref = orc.attn_prefill_i8(qn, qg, kc_ref, vc_ref, pos0, SCALE, nkvh, n_ctx, lo, lo + 4)[lo:lo + 4]
        else:
            ref = orc.attn_ref(qn[lo:lo + 4], qg[lo:lo + 4], kc_ref, vc_ref, pos0 + lo, SCALE, nkvh, n_ctx, q8=True)
        assert_close(out[lo:lo + 4], ref, "prefix %d, tokens %d..%d" % (pos0, lo, lo + 3))
    assert q27.device_status() == 0


def test_prefill_agrees_with_decode(q27, orc):
    """The last 4 tokens of a prefill chunk and a 4-token decode over the same cache differ only by
    the int8 rounding of Q (bounded well inside the path's tolerance)."""
    pos0, M, nkvh = 700, 64, 1
    qn, qg, kc_ref, vc_ref, n, n_ctx = make_case(orc, M, pos0, nkvh)
    kc, vc = dev(kc_ref), dev(vc_ref)
    o = torch.empty((M, 6, AD), device="cuda")
    q27.attn_prefill(dev(qn), dev(qg), kc, vc, o, pos_tensor(pos0), M, SCALE, 6, nkvh, n_ctx)
    o4 = torch.empty((4, 6, AD), device="cuda")
    q27.attn_decode(dev(qn[-4:]), dev(qg[-4:]), kc, vc, o4, None, None, pos_tensor(n - 4), 4, SCALE, 6, nkvh, n_ctx)
    torch.cuda.synchronize()
    assert_close(o[-4:].cpu().numpy(), o4.cpu().numpy(), "prefill vs decode", abs_tol=5e-3, rel_tol=5e-2)


@pytest.mark.parametrize("pos0,M,depth_hint", [(700, 200, -1), (3000, 256, 8192), (0, 129, -1)])
def test_prefill_q8_1_epilogue(q27, orc, pos0, M, depth_hint):
    """With xq the result leaves as q8_1 (what the reference computes with quantize_q8_1 after
    attn_prefill, src/model.cu:1230): exactly the oracle's q8_1 of the kernel's own f32 result, with
    and without the split over the positions (the split path quantises in the merge kernel)."""
    nkvh = 2
    nqh = nkvh * GQA
    qn, qg, kc_ref, vc_ref, n, n_ctx = make_case(orc, M, pos0, nkvh)
    kc, vc = dev(kc_ref), dev(vc_ref)
    o = torch.full((M, nqh, AD), float("nan"), device="cuda")
    q27.attn_prefill(dev(qn), dev(qg), kc, vc, o, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx, True, depth_hint)
    xq = torch.zeros((M, nqh, AD), dtype=torch.int8, device="cuda")
    xd = torch.zeros((M * nqh * 8,), dtype=torch.float32, device="cuda")
    q27.attn_prefill_q8_1(dev(qn), dev(qg), kc, vc, xq, xd, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx, True, depth_hint)
    torch.cuda.synchronize()
    rq, rd = orc.q8_1(o.cpu().numpy().reshape(-1))
    assert np.array_equal(xq.cpu().numpy().reshape(-1), rq)
    assert np.array_equal(xd.cpu().numpy(), rd)
    assert q27.device_status() == 0


@pytest.mark.parametrize("pos0,M,depth_hint", [(0, 37, -1), (0, 128, -1), (1000, 64, -1), (5000, 128, 8000), (63, 2, -1),
                                               (300, 200, -1), (129, 257, 4096)])
def test_prefill_f16_cache(q27, orc, pos0, M, depth_hint):
    """f16 KV cache: the f16-QK kernel (the reference's attn_prefill_kernel<PT, false>,
    src/attn.cu:338-528) against the oracle's statement of the same numerics (Q*scale -> f16, K and V
    as stored, f32 scores, P -> f16), with and without the split over the positions."""
    from qwen27_engine_b200 import synth
    nkvh = 2
    nqh = nkvh * GQA
    n = pos0 + M
    n_ctx = n + 9
    qn = synth.normal(synth.SEED_Q, (M, nqh, AD))
    qg = np.zeros((M, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (M, nqh, AD))
    kf = synth.normal(synth.SEED_K, (nkvh, n, AD))
    vf = synth.normal(synth.SEED_V, (nkvh, n, AD))
    kc_ref, vc_ref = orc.fill_cache(kf, vf, n_ctx, q8=False)
    kc_ref.view(np.uint16).reshape(nkvh, n_ctx, AD)[:, n:] = 0x7E00   # NaN rows past the sequence
    vc_ref.view(np.uint16).reshape(nkvh, n_ctx, AD)[:, n:] = 0x7E00
    o = torch.full((M, nqh, AD), float("nan"), device="cuda")
    q27.attn_prefill(dev(qn), dev(qg), dev(kc_ref), dev(vc_ref), o, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx, False,
                     depth_hint)
    torch.cuda.synchronize()
    ref = orc.attn_ref(qn, qg, kc_ref, vc_ref, pos0, SCALE, nkvh, n_ctx, q8=False)
    assert_close(o.cpu().numpy(), ref, "f16-cache prefill pos0=%d M=%d" % (pos0, M))
    assert q27.device_status() == 0


def test_prefill_f16_cache_q8_1(q27, orc):
    from qwen27_engine_b200 import synth
    nkvh, pos0, M = 1, 500, 130
    nqh = nkvh * GQA
    n = pos0 + M
    n_ctx = n + 5
    qn = synth.normal(synth.SEED_Q, (M, nqh, AD))
    qg = np.zeros((M, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (M, nqh, AD))
    kc_ref, vc_ref = orc.fill_cache(synth.normal(synth.SEED_K, (nkvh, n, AD)), synth.normal(synth.SEED_V, (nkvh, n, AD)),
                                    n_ctx, q8=False)
    kc, vc = dev(kc_ref), dev(vc_ref)
    # the f32 result of the same (split) path, then its q8_1
    o = torch.empty((M, nqh, AD), device="cuda")
    os.environ["Q27_ATTN_SPLIT"] = "2"
    try:
        q27.attn_prefill(dev(qn), dev(qg), kc, vc, o, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx, False, -1)
        xq = torch.zeros((M, nqh, AD), dtype=torch.int8, device="cuda")
        xd = torch.zeros((M * nqh * 8,), dtype=torch.float32, device="cuda")
        q27.attn_prefill_q8_1(dev(qn), dev(qg), kc, vc, xq, xd, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx, False, -1)
        torch.cuda.synchronize()
    finally:
        del os.environ["Q27_ATTN_SPLIT"]
    rq, rd = orc.q8_1(o.cpu().numpy().reshape(-1))
    assert np.array_equal(xq.cpu().numpy().reshape(-1), rq) and np.array_equal(xd.cpu().numpy(), rd)


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("q8", [True, False])
def test_prefill_sharded_over_ranks(q27, orc, world, q8):
    """One chunk shared out by shard.plan_prefill (KV-head groups, then query-token ranges), the ranks
    run one after the other on this GPU: every rank writes its [token][head] slice, nothing is exchanged."""
    from qwen27_engine_b200 import shard, synth
    pos0, M, nkvh = 700, 300, 4
    nqh, n = nkvh * GQA, pos0 + M
    n_ctx = n + 9
    qn = synth.normal(synth.SEED_Q, (M, nqh, AD))
    qg = np.zeros((M, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (M, nqh, AD))
    kf = synth.normal(synth.SEED_K, (nkvh, n, AD))
    vf = synth.normal(synth.SEED_V, (nkvh, n, AD))
    out = np.full((M, nqh, AD), np.nan, np.float32)
    for r in range(world):
        s = shard.plan_prefill(r, world, M, pos0, nkvh)
        h0, nh = s.kv_head0, s.n_kv_heads
        kc, vc = orc.fill_cache(kf[h0:h0 + nh], vf[h0:h0 + nh], n_ctx, q8=q8)
        lq, lg = np.ascontiguousarray(qn[:, h0 * GQA:(h0 + nh) * GQA]), np.ascontiguousarray(qg[:, h0 * GQA:(h0 + nh) * GQA])
        dq, dg, dk, dv = dev(lq), dev(lg), dev(kc), dev(vc)
        o = torch.full((M, nh * GQA, AD), float("nan"), device="cuda")
        for a, b in s.ranges:
            q27.attn_prefill(dq[a:b], dg[a:b], dk, dv, o[a:b], pos_tensor(pos0 + a), b - a, SCALE, nh * GQA, nh, n_ctx, q8,
                             depth_hint=pos0 + a)
        torch.cuda.synchronize()
        got = o.cpu().numpy()
        for a, b in s.ranges:
            assert np.isnan(out[a:b, h0 * GQA:(h0 + nh) * GQA]).all()  # nobody else wrote this slice
            out[a:b, h0 * GQA:(h0 + nh) * GQA] = got[a:b]
    kc, vc = orc.fill_cache(kf, vf, n_ctx, q8=q8)
    ref = orc.attn_prefill_i8(qn, qg, kc, vc, pos0, SCALE, nkvh, n_ctx) if q8 else \
        orc.attn_ref(qn, qg, kc, vc, pos0, SCALE, nkvh, n_ctx, q8=False)
    assert_close(out, ref, "prefill over %d ranks" % world)
    assert q27.device_status() == 0


@pytest.mark.parametrize("q8", [True, False])
def test_prefill_tail_split(q27, orc, q8):
    """More CTAs than SMs on a deep prefix: only the earliest query tile(s) are split over their
    positions and merged, the others write their result directly. Checked on the token ranges around
    the boundary between the two kinds and at the end of the chunk; the q8_1 form of the same call."""
    from qwen27_engine_b200 import synth
    nkvh, pos0, M = 4, 3600, 896      # 7 tiles x 24 heads = 168 CTAs, prefix >= 4 M
    nqh, n = nkvh * GQA, pos0 + M
    n_ctx = n + 9
    qn = synth.normal(synth.SEED_Q, (M, nqh, AD))
    qg = np.zeros((M, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (M, nqh, AD))
    kc_ref, vc_ref = orc.fill_cache(synth.normal(synth.SEED_K, (nkvh, n, AD)), synth.normal(synth.SEED_V, (nkvh, n, AD)),
                                    n_ctx, q8=q8)
    kc, vc = dev(kc_ref), dev(vc_ref)
    o = torch.full((M, nqh, AD), float("nan"), device="cuda")
    q27.attn_prefill(dev(qn), dev(qg), kc, vc, o, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx, q8, pos0)
    torch.cuda.synchronize()
    got = o.cpu().numpy()
    assert np.isfinite(got).all()
    for a, b in [(0, 8), (100, 160), (880, 896)]:
        if q8:
            ref = orc.attn_prefill_i8(qn, qg, kc_ref, vc_ref, pos0, SCALE, nkvh, n_ctx, a, b)[a:b]
        else:
            ref = orc.attn_ref(qn[a:b], qg[a:b], kc_ref, vc_ref, pos0 + a, SCALE, nkvh, n_ctx, q8=False)
        assert_close(got[a:b], ref, "tail split tokens %d..%d" % (a, b))
    if q8:  # unsplit tiles quantise in the kernel's epilogue, split tiles in the merge kernel
        xq = torch.zeros((M, nqh, AD), dtype=torch.int8, device="cuda")
        xd = torch.zeros((M * nqh * 8,), dtype=torch.float32, device="cuda")
        q27.attn_prefill_q8_1(dev(qn), dev(qg), kc, vc, xq, xd, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx, q8, pos0)
        torch.cuda.synchronize()
        rq, rd = orc.q8_1(got.reshape(-1))
        assert np.array_equal(xq.cpu().numpy().reshape(-1), rq) and np.array_equal(xd.cpu().numpy(), rd)
    assert q27.device_status() == 0


@pytest.mark.parametrize("pos0,M,depth_hint", [(0, 37, -1), (0, 128, -1), (1000, 64, -1), (5000, 128, 8000), (63, 2, -1),
                                               (300, 200, -1), (129, 257, 4096)])
def test_prefill_f16_qk_on_q8_cache(q27, orc, pos0, M, depth_hint):
    """q8_0 cache served by the f16-QK kernel (the reference's Q27_ATTN_I8=0, attn_prefill_kernel<PT, true>,
    src/attn.cu:338-528): K and V dequantised to f16 (q * d, one rounding), Q * scale in f16. Cache rows
    past the sequence are poisoned (NaN scales)."""
    nkvh = 2
    nqh = nkvh * GQA
    qn, qg, kc_ref, vc_ref, n, n_ctx = make_case(orc, M, pos0, nkvh)
    o = torch.full((M, nqh, AD), float("nan"), device="cuda")
    q27.set_prefill_kernel(2)
    try:
        q27.attn_prefill(dev(qn), dev(qg), poisoned_cache(q27, kc_ref, nkvh, n_ctx, n),
                         poisoned_cache(q27, vc_ref, nkvh, n_ctx, n), o, pos_tensor(pos0), M, SCALE, nqh, nkvh, n_ctx, True,
                         depth_hint)
        torch.cuda.synchronize()
    finally:
        q27.set_prefill_kernel(0)
    ref = orc.attn_ref(qn, qg, kc_ref, vc_ref, pos0, SCALE, nkvh, n_ctx, q8=True)
    assert_close(o.cpu().numpy(), ref, "f16-QK prefill on q8_0 pos0=%d M=%d" % (pos0, M))
    assert q27.device_status() == 0
