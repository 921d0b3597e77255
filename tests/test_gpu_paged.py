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
