"""The CPU oracle against an independent numpy statement of the same formulas (small cases), and
its internal consistency (partials + merge = whole)."""
import numpy as np
import pytest

from conftest import assert_close

AD, GQA = 256, 6


def np_q8_0(x):
    x = x.astype(np.float32).reshape(-1, 8, 32)
    amax = np.abs(x).max(-1, keepdims=True)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        idv = np.where(d != 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    y = (x * idv).astype(np.float32)
    q = (np.sign(y) * np.floor(np.abs(y) + np.float32(0.5))).astype(np.int8)  # half away from zero
    return q.reshape(-1, AD), d.astype(np.float16).view(np.uint16).reshape(-1, 8)


def np_dequant(q, dbits):
    d = dbits.view(np.float16).astype(np.float32)
    return (q.reshape(-1, 8, 32).astype(np.float32) * d[..., None]).astype(np.float16).astype(np.float32).reshape(-1, AD)


def np_attn(qn, qg, kq, kd, vq, vd, pos0, scale, nkvh, n_ctx):
    T, nqh = qn.shape[:2]
    o = np.zeros((T, nqh, AD), np.float32)
    for t in range(T):
        n = pos0 + t + 1
        for h in range(nqh):
            kh = h // GQA
            K = np_dequant(kq[kh, :n], kd[kh, :n]).astype(np.float64)
            V = np_dequant(vq[kh, :n], vd[kh, :n]).astype(np.float64)
            q = (qn[t, h] * np.float32(scale)).astype(np.float16).astype(np.float64)
            s = (K @ q).astype(np.float32)
            e = np.exp(s - s.max()).astype(np.float32)
            A = e.astype(np.float16).astype(np.float64) @ V
            g = 1.0 / (1.0 + np.exp(-qg[t, h, 256:].astype(np.float64)))
            o[t, h] = (A / e.astype(np.float64).sum()) * g
    return o


def test_q8_0_matches_numpy(orc):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((300, AD)).astype(np.float32)
    x[5] = 0
    x[6, :32] = 0
    x[7] *= 1e-30
    q, d = orc.quant_q8_0(x)
    q2, d2 = np_q8_0(x)
    assert np.array_equal(q, q2) and np.array_equal(d, d2)


def test_cache_layout_and_append(orc):
    rng = np.random.default_rng(2)
    nkvh, n_ctx, T, pos0 = 2, 40, 3, 17
    k = rng.standard_normal((T, nkvh, AD)).astype(np.float32)
    v = rng.standard_normal((T, nkvh, AD)).astype(np.float32)
    for q8 in (True, False):
        kc, vc = orc.new_cache(nkvh, n_ctx, q8, fill=0xAB), orc.new_cache(nkvh, n_ctx, q8, fill=0xAB)
        assert kc.size == nkvh * n_ctx * (272 if q8 else 512)
        orc.kv_append(k, v, kc, vc, pos0, nkvh, n_ctx, q8)
        if q8:
            vals = kc[: nkvh * n_ctx * AD].view(np.int8).reshape(nkvh, n_ctx, AD)
            sc = kc[nkvh * n_ctx * AD:].view(np.uint16).reshape(nkvh, n_ctx, 8)
            for t in range(T):
                for kh in range(nkvh):
                    q, d = np_q8_0(k[t, kh][None])
                    assert np.array_equal(vals[kh, pos0 + t], q[0]) and np.array_equal(sc[kh, pos0 + t], d[0])
            untouched = np.ones(n_ctx, bool)
            untouched[pos0:pos0 + T] = False
            assert (kc[: nkvh * n_ctx * AD].reshape(nkvh, n_ctx, AD)[:, untouched] == 0xAB).all()
        else:
            h = kc.view(np.float16).reshape(nkvh, n_ctx, AD)
            assert np.array_equal(h[:, pos0:pos0 + T], k.transpose(1, 0, 2).astype(np.float16))


@pytest.mark.parametrize("T,n", [(1, 1), (1, 70), (4, 4), (4, 133), (3, 64)])
def test_attn_ref_matches_numpy(orc, T, n):
    rng = np.random.default_rng(3 + n)
    nkvh, nqh, n_ctx = 2, 12, n + 3
    qn = rng.standard_normal((T, nqh, AD)).astype(np.float32)
    qg = rng.standard_normal((T, nqh, 512)).astype(np.float32)
    kf = rng.standard_normal((nkvh, n, AD)).astype(np.float32)
    vf = rng.standard_normal((nkvh, n, AD)).astype(np.float32)
    kc, vc = orc.fill_cache(kf, vf, n_ctx)
    o = orc.attn_ref(qn, qg, kc, vc, n - T, 1 / 16, nkvh, n_ctx)
    kq, kd = np_q8_0(kf)
    vq, vd = np_q8_0(vf)
    ref = np_attn(qn, qg, kq.reshape(nkvh, n, AD), kd.reshape(nkvh, n, 8), vq.reshape(nkvh, n, AD),
                  vd.reshape(nkvh, n, 8), n - T, 1 / 16, nkvh, n_ctx)
    assert_close(o, ref, "attn_ref", abs_tol=5e-5, rel_tol=5e-4)


def test_f16_cache(orc):
    rng = np.random.default_rng(5)
    nkvh, nqh, n, T = 1, 6, 50, 2
    qn = rng.standard_normal((T, nqh, AD)).astype(np.float32)
    qg = rng.standard_normal((T, nqh, 512)).astype(np.float32)
    kf = rng.standard_normal((nkvh, n, AD)).astype(np.float32)
    vf = rng.standard_normal((nkvh, n, AD)).astype(np.float32)
    kc, vc = orc.fill_cache(kf, vf, n, q8=False)
    o = orc.attn_ref(qn, qg, kc, vc, n - T, 1 / 16, nkvh, n, q8=False)
    K, V = kf.astype(np.float16).astype(np.float64), vf.astype(np.float16).astype(np.float64)
    for t in range(T):
        m = n - T + t + 1
        for h in range(nqh):
            q = (qn[t, h] / 16).astype(np.float16).astype(np.float64)
            s = (K[0, :m] @ q).astype(np.float32)
            e = np.exp(s - s.max()).astype(np.float32)
            A = e.astype(np.float16).astype(np.float64) @ V[0, :m]
            ref = A / e.astype(np.float64).sum() / (1 + np.exp(-qg[t, h, 256:].astype(np.float64)))
            assert np.abs(o[t, h] - ref).max() < 2e-5


def test_partials_merge_to_whole(orc):
    rng = np.random.default_rng(7)
    nkvh, nqh, n, T, n_ctx = 2, 12, 300, 4, 320
    qn = rng.standard_normal((T, nqh, AD)).astype(np.float32)
    qg = rng.standard_normal((T, nqh, 512)).astype(np.float32)
    kc, vc = orc.fill_cache(rng.standard_normal((nkvh, n, AD)).astype(np.float32),
                            rng.standard_normal((nkvh, n, AD)).astype(np.float32), n_ctx)
    whole = orc.attn_ref(qn, qg, kc, vc, n - T, 1 / 16, nkvh, n_ctx)
    cuts = [0, 64, 192, 298, 400]
    parts = np.stack([orc.attn_partial(qn, kc, vc, n - T, 1 / 16, nkvh, n_ctx, a, b) for a, b in zip(cuts, cuts[1:])])
    assert parts[-1][3, 0, 0] > -1e29 and parts[-1][0, 0, 0] == np.float32(-1e30)  # causal inside the block
    merged = orc.lse_merge(parts, qg)
    # each slice rounds P to f16 relative to its own maximum: agreement to ~2^-11 relative, not bitwise
    assert_close(merged, whole, "merge", abs_tol=2e-4, rel_tol=2e-3)
    # an empty slice is neutral
    empty = orc.attn_partial(qn, kc, vc, n - T, 1 / 16, nkvh, n_ctx, 300, 320)
    assert (empty[..., 0] == np.float32(-1e30)).all() and (empty[..., 1:] == 0).all()


def test_q8_1(orc):
    rng = np.random.default_rng(8)
    y = rng.standard_normal(32 * 9).astype(np.float32)
    y[32:64] = 0
    xq, xd = orc.q8_1(y)
    for b in range(9):
        blk = y[b * 32:(b + 1) * 32]
        amax = np.abs(blk).max()
        d = np.float32(amax) / np.float32(127)
        assert xd[b] == np.float32(np.float16(d))
        if amax == 0:
            assert (xq[b * 32:(b + 1) * 32] == 0).all()
        else:
            r = (blk / d).astype(np.float32)
            assert np.array_equal(xq[b * 32:(b + 1) * 32], (np.sign(r) * np.floor(np.abs(r) + np.float32(0.5))).astype(np.int8))


def test_prefill_i8_matches_numpy(orc):
    rng = np.random.default_rng(9)
    nkvh, nqh, M, pos0 = 1, 6, 5, 37
    n = pos0 + M
    qn = rng.standard_normal((M, nqh, AD)).astype(np.float32)
    qg = rng.standard_normal((M, nqh, 512)).astype(np.float32)
    kf = rng.standard_normal((nkvh, n, AD)).astype(np.float32)
    vf = rng.standard_normal((nkvh, n, AD)).astype(np.float32)
    kc, vc = orc.fill_cache(kf, vf, n)
    o = orc.attn_prefill_i8(qn, qg, kc, vc, pos0, 1 / 16, nkvh, n)
    kq, kd = np_q8_0(kf)
    vq, vd = np_q8_0(vf)
    V = np_dequant(vq, vd).astype(np.float64)
    dk = kd.view(np.float16).astype(np.float32)
    q8, dq = orc.quant_q_i8(qn, 1 / 16)
    # the integer stage against plain integer arithmetic
    acc = orc.qk_i32(q8[0], kq)
    ref_acc = np.einsum("hbi,pbi->hpb", q8[0].reshape(nqh, 8, 32).astype(np.int64), kq.reshape(n, 8, 32).astype(np.int64))
    assert np.array_equal(acc, ref_acc.astype(np.int32))
    # the int8 quantiser: round half to even of v * (127 / amax)
    v = (qn * np.float32(1 / 16)).astype(np.float32).reshape(M, nqh, 8, 32)
    amax = np.abs(v).max(-1, keepdims=True)
    assert np.array_equal(q8.reshape(M, nqh, 8, 32), np.rint(v * (np.float32(127) / amax)).astype(np.int8))
    assert np.array_equal(dq, (amax[..., 0] / np.float32(127)).astype(np.float32))
    for t in range(M):
        m = pos0 + t + 1
        for h in range(nqh):
            I = np.einsum("bi,pbi->pb", q8[t, h].reshape(8, 32).astype(np.int64), kq[:m].reshape(m, 8, 32).astype(np.int64))
            s = np.zeros(m, np.float32)
            for b in range(8):
                s += (dq[t, h, b] * dk[:m, b]).astype(np.float32) * I[:, b].astype(np.float32)
            e = np.exp(s - s.max()).astype(np.float32)
            A = e.astype(np.float16).astype(np.float64) @ V[:m]
            ref = A / e.astype(np.float64).sum() / (1 + np.exp(-qg[t, h, 256:].astype(np.float64)))
            assert np.abs(o[t, h] - ref).max() < 2e-5


def test_kv_wire_layout_round_trip(orc):
    """Reference host layout of cache rows (Decoder::kv_copy, src/model.cu:1809-1830): values of all
    heads first, then the scales; packing and unpacking are inverse and touch only rows [p0, p1)."""
    rng = np.random.default_rng(5)
    nkvh, n_ctx, p0, p1 = 3, 50, 7, 31
    cache = rng.integers(0, 256, orc.kv_cache_bytes(nkvh, n_ctx, True), dtype=np.uint8)
    wire = orc.kv_wire_from_cache(cache, nkvh, n_ctx, p0, p1)
    n = p1 - p0
    assert wire.size == nkvh * n * 272
    # head 1, row p0 + 2: its 256 value bytes and its 16 scale bytes
    assert np.array_equal(wire[(1 * n + 2) * 256:(1 * n + 3) * 256], cache[(1 * n_ctx + p0 + 2) * 256:(1 * n_ctx + p0 + 3) * 256])
    s0 = nkvh * n_ctx * 256
    assert np.array_equal(wire[nkvh * n * 256 + (1 * n + 2) * 16:nkvh * n * 256 + (1 * n + 3) * 16],
                          cache[s0 + (1 * n_ctx + p0 + 2) * 16:s0 + (1 * n_ctx + p0 + 3) * 16])
    other = np.zeros_like(cache)
    orc.kv_wire_to_cache(other, wire, nkvh, n_ctx, p0, p1)
    assert np.array_equal(orc.kv_wire_from_cache(other, nkvh, n_ctx, p0, p1), wire)
    mask = np.ones(cache.size, bool)
    vals = mask[:s0].reshape(nkvh, n_ctx, 256); vals[:, p0:p1] = False
    sc = mask[s0:].reshape(nkvh, n_ctx, 16); sc[:, p0:p1] = False
    assert (other[mask] == 0).all()
