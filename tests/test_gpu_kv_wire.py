"""KV rows between the caches and the reference's host layout (Decoder::kv_copy, src/model.cu:1809-1830):
byte-exact against the oracle's restatement, page pool and contiguous cache, both directions."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from helpers_gpu import dev
from test_gpu_paged import build_pool

pytestmark = pytest.mark.gpu
AD, GQA, PAGE = 256, 6, 256
SCALE = 1.0 / 16.0


def _sequence(orc, nkvh, n, seed_shift=0):
    from qwen27_engine_b200 import synth
    kf = synth.normal(synth.SEED_K, (nkvh, n, AD), start=seed_shift << 24)
    vf = synth.normal(synth.SEED_V, (nkvh, n, AD), start=seed_shift << 24)
    return kf, vf


@pytest.mark.parametrize("nkvh,n,p0,p1", [(2, 1000, 0, 1000), (4, 3000, 255, 2049), (1, 300, 299, 300), (2, 70000, 0, 70000)])
def test_pages_to_wire_matches_the_reference_layout(q27, orc, nkvh, n, p0, p1):
    from qwen27_engine_b200 import synth
    kf, _ = _sequence(orc, nkvh, n)
    need = (n + PAGE - 1) // PAGE
    n_pages = need + 5
    table = synth.permutation(synth.SEED_LEN, n_pages)[:need].astype(np.int32)
    pool = build_pool(orc, [kf], nkvh, n_pages, [table])
    kc, _ = orc.fill_cache(kf, kf, n)                      # the same rows in a contiguous cache, n_ctx = n
    want = orc.kv_wire_from_cache(kc, nkvh, n, p0, p1)
    assert want.size == q27.kv_wire_bytes(nkvh, p1 - p0)
    wire = torch.full((want.size,), 0xA5, dtype=torch.uint8, device="cuda")
    q27.kv_pages_to_wire(dev(pool), dev(table), wire, nkvh, n_pages, p0, p1)
    torch.cuda.synchronize()
    assert np.array_equal(wire.cpu().numpy(), want)
    # and from the contiguous cache, which is what the reference's two strided copies produce
    wire2 = torch.full((want.size,), 0x5A, dtype=torch.uint8, device="cuda")
    q27.kv_cache_to_wire(dev(kc), wire2, nkvh, n, p0, p1)
    torch.cuda.synchronize()
    assert np.array_equal(wire2.cpu().numpy(), want)
    assert q27.device_status() == 0


def test_swap_out_paged_restore_contiguous_and_back(q27, orc):
    """A sequence written into pages is packed, restored into a contiguous cache and decoded there;
    then packed from the contiguous cache and scattered into other pages: same bytes, same attention."""
    from qwen27_engine_b200 import synth
    nkvh, n, T = 2, 2500, 4
    nqh = nkvh * GQA
    kf, vf = _sequence(orc, nkvh, n, 3)
    need = (n + PAGE - 1) // PAGE
    n_pages = 2 * need + 3
    perm = synth.permutation(synth.SEED_LEN, n_pages).astype(np.int32)
    tab_a, tab_b = perm[:need], perm[need:2 * need]
    kpool, vpool = dev(build_pool(orc, [kf], nkvh, n_pages, [tab_a])), dev(build_pool(orc, [vf], nkvh, n_pages, [tab_a]))
    nbytes = q27.kv_wire_bytes(nkvh, n)
    kw = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    vw = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    q27.kv_pages_to_wire(kpool, dev(tab_a), kw, nkvh, n_pages, 0, n)
    q27.kv_pages_to_wire(vpool, dev(tab_a), vw, nkvh, n_pages, 0, n)
    host_k, host_v = kw.cpu(), vw.cpu()                      # "swapped out": one contiguous copy each
    n_ctx = n + 37
    kc, vc = q27.new_cache(nkvh, n_ctx), q27.new_cache(nkvh, n_ctx)
    q27.kv_wire_to_cache(kc, host_k.cuda(), nkvh, n_ctx, 0, n)
    q27.kv_wire_to_cache(vc, host_v.cuda(), nkvh, n_ctx, 0, n)
    kc_ref, vc_ref = orc.fill_cache(kf, vf, n_ctx)
    qn = synth.normal(synth.SEED_Q, (T, nqh, AD))
    qg = np.zeros((T, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (T, nqh, AD))
    o = torch.full((T, nqh, AD), float("nan"), device="cuda")
    pos = torch.tensor([n - T], dtype=torch.int32, device="cuda")
    q27.attn_decode(dev(qn), dev(qg), kc, vc, o, None, None, pos, T, SCALE, nqh, nkvh, n_ctx)
    torch.cuda.synchronize()
    ref = orc.attn_ref(qn, qg, kc_ref, vc_ref, n - T, SCALE, nkvh, n_ctx)
    assert_close(o.cpu().numpy(), ref, "decode on the restored contiguous cache")
    # back into other pages of the pool, through the wire layout again
    q27.kv_cache_to_wire(kc, kw, nkvh, n_ctx, 0, n)
    q27.kv_cache_to_wire(vc, vw, nkvh, n_ctx, 0, n)
    assert torch.equal(kw.cpu(), host_k) and torch.equal(vw.cpu(), host_v)
    q27.kv_wire_to_pages(kpool, dev(tab_b), kw, nkvh, n_pages, 0, n)
    q27.kv_wire_to_pages(vpool, dev(tab_b), vw, nkvh, n_pages, 0, n)
    tables = np.full((1, need), -1, np.int32)
    tables[0] = tab_b
    o2 = torch.full((1, T, nqh, AD), float("nan"), device="cuda")
    q27.attn_decode_paged(dev(qn[None]), dev(qg[None]), kpool, vpool, dev(tables), dev(np.array([n], np.int32)), o2, 1, T,
                          SCALE, nqh, nkvh, n_pages, need, n)
    torch.cuda.synchronize()
    assert_close(o2.cpu().numpy()[0], ref, "paged decode on the re-scattered pages")
    assert q27.device_status() == 0


def test_bad_page_is_flagged_and_skipped(q27):
    nkvh, n_pages = 1, 4
    pool = torch.zeros(q27.kv_pool_bytes(nkvh, n_pages), dtype=torch.uint8, device="cuda")
    wire = torch.full((q27.kv_wire_bytes(nkvh, 300),), 7, dtype=torch.uint8, device="cuda")
    q27.kv_pages_to_wire(pool, dev(np.array([0, 999], np.int32)), wire, nkvh, n_pages, 0, 300)
    assert q27.device_status() & 2
    w = wire.cpu().numpy()
    assert (w[:256 * AD] == 0).all() and (w[256 * AD:300 * AD] == 7).all()  # rows of the bad page were left alone
