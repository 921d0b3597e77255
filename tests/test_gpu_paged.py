"""Batched decode over the paged q8_0 cache (256-position pages, random page table)."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from helpers_gpu import dev

pytestmark = pytest.mark.gpu
AD, GQA, PAGE = 256, 6, 256
SCALE = 1.0 / 16.0


@pytest.fixture(autouse=True, params=[1, 2, 3, 4], ids=["mma", "tc", "ws", "wt"])
def decode_kernel(request, q27):
    """Every test of this module runs on every split-K kernel (warp-MMA, tcgen05, warp-specialised, warp-specialised with P V on tcgen05)."""
    q27.set_decode_kernel(request.param)
    yield request.param
    q27.set_decode_kernel(0)


def build_pool(orc, kfs, nkvh, n_pages, tables):
    """Scatters each sequence's q8_0 rows into a pool [n_pages][nkvh][256] rows (+ scales)."""
    vals = np.full((n_pages, nkvh, PAGE, AD), 0x7F, np.uint8)
    sc = np.full((n_pages, nkvh, PAGE, 8), 0xFFFF, np.uint16)  # NaN scales wherever nothing was written
    for kf, tab in zip(kfs, tables):
        q, d = orc.quant_q8_0(kf)  # [nkvh][n][256]
        n = kf.shape[1]
        for j in range((n + PAGE - 1) // PAGE):
            m = min(PAGE, n - j * PAGE)
            vals[tab[j], :, :m] = q[:, j * PAGE:j * PAGE + m].view(np.uint8)
            sc[tab[j], :, :m] = d[:, j * PAGE:j * PAGE + m]
    return np.concatenate([vals.reshape(-1), sc.reshape(-1).view(np.uint8)])


@pytest.mark.parametrize("T,lens", [(4, [300, 5, 4096, 1025, 777]), (1, [1, 256, 257, 9000]), (4, [20000, 1024, 131])])
def test_paged_batched_decode(q27, orc, T, lens):
    from qwen27_engine_b200 import synth
    nkvh = 2
    nqh = nkvh * GQA
    B = len(lens)
    max_len = max(lens)
    max_pages = (max_len + PAGE - 1) // PAGE
    need = sum((n + PAGE - 1) // PAGE for n in lens)
    n_pages = need + 3
    perm = synth.permutation(synth.SEED_LEN, n_pages)
    tables = np.full((B, max_pages), -1, np.int32)
    at = 0
    for b, n in enumerate(lens):
        k = (n + PAGE - 1) // PAGE
        tables[b, :k] = perm[at:at + k]
        at += k
    qn = synth.normal(synth.SEED_Q, (B, T, nqh, AD))
    qg = np.zeros((B, T, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (B, T, nqh, AD))
    kfs = [synth.normal(synth.SEED_K, (nkvh, n, AD), start=b << 24) for b, n in enumerate(lens)]
    vfs = [synth.normal(synth.SEED_V, (nkvh, n, AD), start=b << 24) for b, n in enumerate(lens)]
    kpool = build_pool(orc, kfs, nkvh, n_pages, tables)
    vpool = build_pool(orc, vfs, nkvh, n_pages, tables)
    assert kpool.size == q27.kv_pool_bytes(nkvh, n_pages)
    o = torch.full((B, T, nqh, AD), float("nan"), device="cuda")
    q27.attn_decode_paged(dev(qn), dev(qg), dev(kpool), dev(vpool), dev(tables), dev(np.array(lens, np.int32)), o, B, T,
                          SCALE, nqh, nkvh, n_pages, max_pages, max_len)
    torch.cuda.synchronize()
    out = o.cpu().numpy()
    for b, n in enumerate(lens):
        kc, vc = orc.fill_cache(kfs[b], vfs[b], n)
        ref = orc.attn_ref(qn[b], qg[b], kc, vc, n - T, SCALE, nkvh, n)
        assert_close(out[b], ref, "sequence %d (len %d)" % (b, n))
    assert q27.device_status() == 0


def test_bad_page_is_flagged_not_followed(q27, orc):
    nkvh, nqh, T, n = 1, 6, 1, 300
    n_pages = 4
    pool = torch.zeros(q27.kv_pool_bytes(nkvh, n_pages), dtype=torch.uint8, device="cuda")
    tables = np.array([[0, 999]], np.int32)  # second page index is outside the pool
    o = torch.empty((1, T, nqh, AD), device="cuda")
    q27.attn_decode_paged(torch.zeros((1, T, nqh, AD), device="cuda"), torch.zeros((1, T, nqh, 512), device="cuda"),
                          pool, pool, dev(tables), dev(np.array([n], np.int32)), o, 1, T, SCALE, nqh, nkvh, n_pages, 2, n)
    torch.cuda.synchronize()
    assert q27.device_status() == 2  # ST_BAD_PAGE
    assert q27.device_status() == 0  # reading clears it


def test_config5_at_full_size(q27, orc):
    """The batched configuration of the metric at its real size: 64 sequences of 4 query tokens, lengths
    uniform in 1,024..131,072 (seed 1005), 24 Q / 4 KV heads, 256-token pages behind a random page table
    (10 GB of K and V). The pool is filled on the device (int8 values of the spread that q8_0 gives N(0,1)
    rows, scales around 1/50); for the shortest, the longest and four more sequences the pages are read
    back, put in order and given to the oracle."""
    T, nkvh, B = 4, 4, 64
    nqh = nkvh * GQA
    rng = np.random.default_rng(1005)
    lens = rng.integers(1024, 131072 + 1, size=B)
    max_pages = (131072 + PAGE - 1) // PAGE
    need = [(int(n) + PAGE - 1) // PAGE for n in lens]
    n_pages = sum(need)
    perm = rng.permutation(n_pages).astype(np.int32)
    tables = np.full((B, max_pages), -1, np.int32)
    at = 0
    for b in range(B):
        tables[b, :need[b]] = perm[at:at + need[b]]
        at += need[b]
    g = torch.Generator(device="cuda")
    g.manual_seed(1005)
    nval, nsc = n_pages * nkvh * PAGE * AD, n_pages * nkvh * PAGE * 8

    def pool():
        buf = torch.empty(q27.kv_pool_bytes(nkvh, n_pages), dtype=torch.uint8, device="cuda")
        step = 1 << 28
        for a in range(0, nval, step):
            m = min(step, nval - a)
            v = (torch.randn((m,), generator=g, device="cuda") * 42.0).round_().clamp_(-127, 127).to(torch.int8)
            buf[a:a + m] = v.view(torch.uint8)
        sc = (torch.rand((nsc,), generator=g, device="cuda") * 0.01 + 0.015).to(torch.float16)
        buf[nval:nval + 2 * nsc] = sc.view(torch.uint8)
        return buf
    kpool, vpool = pool(), pool()
    qn = torch.randn((B, T, nqh, AD), generator=g, device="cuda")
    qg = torch.randn((B, T, nqh, 512), generator=g, device="cuda")
    o = torch.full((B, T, nqh, AD), float("nan"), device="cuda")
    q27.attn_decode_paged(qn, qg, kpool, vpool, dev(tables), dev(lens.astype(np.int32)), o, B, T, SCALE, nqh, nkvh,
                          n_pages, max_pages, int(lens.max()))
    torch.cuda.synchronize()
    assert q27.device_status() == 0
    out = o.cpu().numpy()
    assert np.isfinite(out).all()
    order = np.argsort(lens)
    sample = sorted({int(order[0]), int(order[-1]), int(order[B // 5]), int(order[B // 2]), int(order[3 * B // 4]), 0})
    assert len(sample) >= 5

    def gather(pool_t, b):
        """The oracle's contiguous cache [nkvh][n][256] + scales of sequence b, from its pages."""
        n = int(lens[b])
        pages = torch.from_numpy(tables[b, :need[b]].astype(np.int64)).cuda()
        vals = pool_t[:nval].view(n_pages, nkvh, PAGE, AD)[pages].permute(1, 0, 2, 3).reshape(nkvh, -1, AD)[:, :n]
        sc = pool_t[nval:nval + 2 * nsc].view(n_pages, nkvh, PAGE, 16)[pages].permute(1, 0, 2, 3).reshape(nkvh, -1, 16)[:, :n]
        return np.concatenate([vals.contiguous().cpu().numpy().reshape(-1), sc.contiguous().cpu().numpy().reshape(-1)])
    qn_h, qg_h = qn.cpu().numpy(), qg.cpu().numpy()
    for b in sample:
        n = int(lens[b])
        ref = orc.attn_ref(qn_h[b], qg_h[b], gather(kpool, b), gather(vpool, b), n - T, SCALE, nkvh, n)
        assert_close(out[b], ref, "sequence %d of 64 (len %d)" % (b, n))


def _pool_rows(pool, nkvh, n_pages, page, rows):
    """Bytes of the first `rows` rows of a page (all heads): values [nkvh][rows][256], scales [nkvh][rows][16]."""
    nval = n_pages * nkvh * PAGE * AD
    vals = pool[:nval].view(n_pages, nkvh, PAGE, AD)[page, :, :rows].cpu().numpy()
    sc = pool[nval:].view(n_pages, nkvh, PAGE, 16)[page, :, :rows].cpu().numpy()
    return vals, sc


@pytest.mark.parametrize("norm", [False, True])
def test_prep_paged_equals_prep_per_sequence(q27, norm):
    """The batched prologue over the page pool writes, row for row, the bytes that attn_prep writes into a
    contiguous cache of each sequence, and the same qn; nothing else in the pool changes."""
    rng = np.random.default_rng(5)
    T, nkvh, B = 4, 2, 3
    nqh = nkvh * GQA
    lens = [4, 259, 700]  # the new tokens included: rows 0..3, 255..258 (across a page boundary), 696..699
    max_pages = 4
    pager = q27.Pager(12, B, max_pages)
    seqs = [pager.open() for _ in range(B)]
    for s, n in zip(reversed(seqs), reversed(lens)):  # not in order: page numbers differ from a plain count
        pager.extend(s, n)
    table, seq_len = pager.tables(seqs)
    n_pages = pager.n_pages
    qg = rng.standard_normal((B, T, nqh, 512)).astype(np.float32)
    k = rng.standard_normal((B, T, nkvh, AD)).astype(np.float32)
    v = (rng.standard_normal((B, T, nkvh, AD)) * 2).astype(np.float32)
    qw = (1 + 0.1 * rng.standard_normal(AD)).astype(np.float32)
    kw = (1 + 0.1 * rng.standard_normal(AD)).astype(np.float32)
    eps, theta_scale = 1e-6, float(10000000.0 ** (-2.0 / 64))
    rdelta = np.array([0, 3, 1], np.int32)
    kpool = torch.full((q27.kv_pool_bytes(nkvh, n_pages),), 0xAB, dtype=torch.uint8, device="cuda")
    vpool = torch.full((q27.kv_pool_bytes(nkvh, n_pages),), 0xAB, dtype=torch.uint8, device="cuda")
    qn = torch.full((B, T, nqh, AD), float("nan"), device="cuda")
    q27.attn_prep_paged(dev(qg) if norm else None, dev(k), dev(v), dev(qw) if norm else None, dev(kw) if norm else None,
                        qn if norm else None, kpool, vpool, dev(table), dev(seq_len), B, T, eps, theta_scale, nqh, nkvh,
                        n_pages, max_pages, rdelta=dev(rdelta) if norm else None)
    torch.cuda.synchronize()
    assert q27.device_status() == 0
    touched = set()
    for b, n in enumerate(lens):
        n_ctx = n
        kc, vc = q27.new_cache(nkvh, n_ctx, True, fill=0xAB), q27.new_cache(nkvh, n_ctx, True, fill=0xAB)
        if norm:
            qn1 = torch.empty((T, nqh, AD), device="cuda")
            q27.attn_prep(dev(qg[b]), dev(k[b]), dev(v[b]), dev(qw), dev(kw), qn1, kc, vc,
                          dev(np.array([n - T], np.int32)), T, eps, theta_scale, nqh, nkvh, n_ctx,
                          rdelta=dev(rdelta[b:b + 1]))
            assert torch.equal(qn1, qn[b])
        else:
            q27.kv_append(dev(k[b]), dev(v[b]), kc, vc, dev(np.array([n - T], np.int32)), T, nkvh, n_ctx, True)
        torch.cuda.synchronize()
        for cache, pool in ((kc, kpool), (vc, vpool)):
            cv = cache[:nkvh * n_ctx * AD].view(nkvh, n_ctx, AD).cpu().numpy()
            cs = cache[nkvh * n_ctx * AD:].view(nkvh, n_ctx, 16).cpu().numpy()
            for pos in range(n - T, n):
                page, row = int(table[b, pos // PAGE]), pos % PAGE
                touched.add((page, row))
                pv, ps = _pool_rows(pool, nkvh, n_pages, page, PAGE)
                assert np.array_equal(pv[:, row], cv[:, pos]) and np.array_equal(ps[:, row], cs[:, pos])
    # every other row of the pool still holds the canary
    nval = n_pages * nkvh * PAGE * AD
    vals = kpool[:nval].view(n_pages, nkvh, PAGE, AD).cpu().numpy()
    mask = np.ones((n_pages, PAGE), bool)
    for page, row in touched:
        mask[page, row] = False
    assert (vals.transpose(0, 2, 1, 3)[mask] == 0xAB).all()


def test_bad_page_in_prep_is_flagged(q27):
    nkvh, T = 1, 2
    pool = torch.full((q27.kv_pool_bytes(nkvh, 2),), 0xAB, dtype=torch.uint8, device="cuda")
    k = torch.ones((1, T, nkvh, AD), device="cuda")
    q27.attn_prep_paged(None, k, k, None, None, None, pool, pool, dev(np.array([[5, -1]], np.int32)),
                        dev(np.array([T], np.int32)), 1, T, 0.0, 1.0, 6, nkvh, 2, 2)
    torch.cuda.synchronize()
    assert q27.device_status() == 2  # ST_BAD_PAGE
    assert (pool.cpu().numpy() == 0xAB).all()


def test_pager_fork_append_decode(q27, orc):
    """A sequence and a fork of it that shares its first pages, both continued with different tokens through
    attn_prep_paged (append only), give the attention of their own token streams."""
    from qwen27_engine_b200 import synth
    T, nkvh = 4, 2
    nqh = nkvh * GQA
    max_pages, n_pages = 6, 16
    pager = q27.Pager(n_pages, 4, max_pages)
    kpool = torch.full((q27.kv_pool_bytes(nkvh, n_pages),), 0x7F, dtype=torch.uint8, device="cuda")
    vpool = torch.full((q27.kv_pool_bytes(nkvh, n_pages),), 0x7F, dtype=torch.uint8, device="cuda")

    def append(seq, kf, vf):
        """kf, vf [nkvh][m][256]: m more tokens of sequence `seq`."""
        m = kf.shape[1]
        pager.extend(seq, pager.length(seq) + m)
        table, lens = pager.tables([seq])
        k = np.ascontiguousarray(kf.transpose(1, 0, 2))[None]
        v = np.ascontiguousarray(vf.transpose(1, 0, 2))[None]
        q27.attn_prep_paged(None, dev(k), dev(v), None, None, None, kpool, vpool, dev(table), dev(lens), 1, m, 0.0, 1.0,
                            nqh, nkvh, n_pages, max_pages)

    n0, fork_at, n_a, n_b = 600, 530, 300, 90
    k0, v0 = synth.normal(synth.SEED_K, (nkvh, n0, AD)), synth.normal(synth.SEED_V, (nkvh, n0, AD))
    ka, va = synth.normal(synth.SEED_K, (nkvh, n_a, AD), start=1 << 24), synth.normal(synth.SEED_V, (nkvh, n_a, AD), start=1 << 24)
    kb, vb = synth.normal(synth.SEED_K, (nkvh, n_b, AD), start=2 << 24), synth.normal(synth.SEED_V, (nkvh, n_b, AD), start=2 << 24)
    a = pager.open()
    append(a, k0, v0)
    b, cp = pager.fork(a, fork_at)
    assert cp is not None and cp[2] == fork_at % PAGE
    q27.kv_page_copy(kpool, *cp, nkvh, n_pages)
    q27.kv_page_copy(vpool, *cp, nkvh, n_pages)
    append(a, ka, va)   # a = k0 + ka
    append(b, kb, vb)   # b = k0[:fork_at] + kb
    table, lens = pager.tables([a, b])
    assert list(lens) == [n0 + n_a, fork_at + n_b] and list(table[0, :2]) == list(table[1, :2]) and table[0, 2] != table[1, 2]
    qn = synth.normal(synth.SEED_Q, (2, T, nqh, AD))
    qg = np.zeros((2, T, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (2, T, nqh, AD))
    o = torch.full((2, T, nqh, AD), float("nan"), device="cuda")
    q27.attn_decode_paged(dev(qn), dev(qg), kpool, vpool, dev(table), dev(lens), o, 2, T, SCALE, nqh, nkvh, n_pages,
                          max_pages, int(lens.max()))
    torch.cuda.synchronize()
    assert q27.device_status() == 0
    out = o.cpu().numpy()
    streams = [(np.concatenate([k0, ka], 1), np.concatenate([v0, va], 1)),
               (np.concatenate([k0[:, :fork_at], kb], 1), np.concatenate([v0[:, :fork_at], vb], 1))]
    for i, (kf, vf) in enumerate(streams):
        n = kf.shape[1]
        kc, vc = orc.fill_cache(kf, vf, n)
        ref = orc.attn_ref(qn[i], qg[i], kc, vc, n - T, SCALE, nkvh, n)
        assert_close(out[i], ref, "sequence %d (len %d)" % (i, n))
    # cut the fork back below the fork point and let it grow again: it needs its own copy of the shared page first
    pager.cut(b, 300)
    cp2 = pager.unshare(b)
    assert cp2 is not None and cp2[2] == 300 - PAGE
    q27.kv_page_copy(kpool, *cp2, nkvh, n_pages)
    q27.kv_page_copy(vpool, *cp2, nkvh, n_pages)
    append(b, kb, vb)   # b = k0[:300] + kb; a is untouched
    table, lens = pager.tables([a, b])
    q27.attn_decode_paged(dev(qn), dev(qg), kpool, vpool, dev(table), dev(lens), o, 2, T, SCALE, nqh, nkvh, n_pages,
                          max_pages, int(lens.max()))
    torch.cuda.synchronize()
    out = o.cpu().numpy()
    streams[1] = (np.concatenate([k0[:, :300], kb], 1), np.concatenate([v0[:, :300], vb], 1))
    for i, (kf, vf) in enumerate(streams):
        n = kf.shape[1]
        kc, vc = orc.fill_cache(kf, vf, n)
        ref = orc.attn_ref(qn[i], qg[i], kc, vc, n - T, SCALE, nkvh, n)
        assert_close(out[i], ref, "after the cut: sequence %d (len %d)" % (i, n))
