"""The CPU oracle against tests/golden/ref_b200.npz: outputs of the reference's own kernels
(compiled for sm_100a, run on a B200 by tests/golden/make_golden.py) on the same seeded inputs.
This is what pins the oracle; the GPU tests then compare the new kernels with the oracle, and the
last test here compares them with the fixture directly."""
import os

import numpy as np
import pytest

from conftest import ROOT, assert_close, err_stats
from golden_cases import CASES, case_inputs

AD = 256
PATH = os.path.join(ROOT, "tests", "golden", "ref_b200.npz")


@pytest.fixture(scope="module")
def gold(q27):
    assert os.path.exists(PATH), "golden fixture missing: run tests/golden/make_golden.py on a B200"
    return np.load(PATH)


def split_q8(cache, nkvh, n_ctx):
    vals = cache[: nkvh * n_ctx * AD].view(np.int8).reshape(nkvh, n_ctx, AD)
    sc = cache[nkvh * n_ctx * AD:].view(np.float16).reshape(nkvh, n_ctx, 8)
    return vals, sc


def test_q8_0_quantiser_against_reference_bytes(gold, orc):
    """V rows are written raw by the reference's attn_prep: its bytes are the q8_0 quantiser's
    output. The reference is built with fast-math (approximate division), the oracle is IEEE: a
    value that sits on a rounding boundary may differ by one step; everything else is identical."""
    total = bad = 0
    for name in ("prep_q8", "prep_q8_many"):
        c = CASES[name]
        x = case_inputs(name)
        T, nkvh, n_ctx, pos0 = c["T"], c["nkvh"], c["n_ctx"], c["pos0"]
        kc, vc = orc.new_cache(nkvh, n_ctx), orc.new_cache(nkvh, n_ctx)
        orc.kv_append(x["k"], x["v"], kc, vc, pos0, nkvh, n_ctx)
        rv, rs = split_q8(gold[name + "/vcache"], nkvh, n_ctx)
        ov, os_ = split_q8(vc, nkvh, n_ctx)
        d = np.abs(rv.astype(np.int32) - ov.astype(np.int32))
        assert d.max() <= 1
        total += d.size
        bad += int((d != 0).sum())
        sd = np.abs(rs.astype(np.float32) - os_.astype(np.float32))
        assert (sd <= np.abs(os_.astype(np.float32)) * 2.0 ** -10).all()  # at most one f16 ulp
        untouched = np.ones(n_ctx, bool)
        untouched[pos0:pos0 + T] = False
        assert (rv[:, untouched] == 0).all()
    assert bad <= 1e-4 * total, "%d of %d values differ" % (bad, total)


def test_f16_cache_rows(gold, orc):
    c = CASES["prep_f16"]
    x = case_inputs("prep_f16")
    kc, vc = orc.new_cache(c["nkvh"], c["n_ctx"], False), orc.new_cache(c["nkvh"], c["n_ctx"], False)
    orc.kv_append(x["k"], x["v"], kc, vc, c["pos0"], c["nkvh"], c["n_ctx"], False)
    assert np.array_equal(gold["prep_f16/vcache"], vc)


@pytest.mark.parametrize("name", ["decode_cfg1", "decode_t4", "decode_f16"])
def test_decode_oracle_against_reference_kernels(gold, orc, name):
    c = CASES[name]
    x = case_inputs(name)
    kc, vc = orc.fill_cache(x["k"], x["v"], c["n_ctx"], c["q8"])
    o = orc.attn_ref(x["qn"], x["qg"], kc, vc, c["n"] - c["T"], c["scale"], c["nkvh"], c["n_ctx"], c["q8"])
    # the reference's slow kernel is the definition: agreement far inside the path's tolerance
    assert_close(o, gold[name + "/slow"], name + " vs attn_decode_ref", abs_tol=5e-5, rel_tol=1e-3)
    # its fast kernel (online softmax, mma.sync) within the tolerance of the path
    assert_close(o, gold[name + "/fast"], name + " vs attn_decode")


def test_q8_1_epilogue_against_reference(gold, orc):
    """The reference's fused q8_1 output equals the oracle's q8_1 of the reference's own f32 output,
    except where fast-math division moves a value across a rounding boundary."""
    xq, xd = orc.q8_1(gold["decode_t4/fast"].reshape(-1))
    d = np.abs(xq.astype(np.int32) - gold["decode_t4/xq"].reshape(-1).astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() <= 2e-3
    assert np.abs(xd - gold["decode_t4/xd"]).max() <= np.abs(xd).max() * 2.0 ** -10


@pytest.mark.parametrize("name", ["prefill_a", "prefill_b"])
def test_prefill_oracle_against_reference_kernel(gold, orc, name):
    c = CASES[name]
    x = case_inputs(name)
    kc, vc = orc.fill_cache(x["k"], x["v"], c["n_ctx"], True)
    o = orc.attn_prefill_i8(x["qn"], x["qg"], kc, vc, c["pos0"], c["scale"], c["nkvh"], c["n_ctx"])
    # the reference kernel accumulates O in f16 (its own source of error): tolerance of the path
    assert_close(o, gold[name + "/i8"], name + " vs attn_prefill (int8)")
    # and the int8 rounding of Q stays close to the f16-Q definition
    mx, rms, l2 = err_stats(o, gold[name + "/slow_f16q"])
    assert l2 <= 2e-2


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["decode_cfg1", "decode_t4"])
def test_new_decode_kernel_against_reference_outputs(gold, q27, orc, name):
    import torch
    from helpers_gpu import dev, pos_tensor
    c = CASES[name]
    x = case_inputs(name)
    nqh = c["nkvh"] * 6
    kc, vc = orc.fill_cache(x["k"], x["v"], c["n_ctx"], True)
    o = torch.empty((c["T"], nqh, AD), device="cuda")
    q27.attn_decode(dev(x["qn"]), dev(x["qg"]), dev(kc), dev(vc), o, None, None, pos_tensor(c["n"] - c["T"]), c["T"],
                    c["scale"], nqh, c["nkvh"], c["n_ctx"])
    torch.cuda.synchronize()
    assert_close(o.cpu().numpy(), gold[name + "/slow"], name + ": new kernel vs the reference's slow kernel")
    assert_close(o.cpu().numpy(), gold[name + "/fast"], name + ": new kernel vs the reference's fast kernel")


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["prefill_a", "prefill_b"])
def test_new_prefill_kernel_against_reference_outputs(gold, q27, orc, name):
    import torch
    from helpers_gpu import dev, pos_tensor
    c = CASES[name]
    x = case_inputs(name)
    nqh = c["nkvh"] * 6
    kc, vc = orc.fill_cache(x["k"], x["v"], c["n_ctx"], True)
    o = torch.empty((c["M"], nqh, AD), device="cuda")
    q27.attn_prefill(dev(x["qn"]), dev(x["qg"]), dev(kc), dev(vc), o, pos_tensor(c["pos0"]), c["M"], c["scale"], nqh,
                     c["nkvh"], c["n_ctx"])
    torch.cuda.synchronize()
    assert_close(o.cpu().numpy(), gold[name + "/i8"], name + ": new kernel vs the reference's int8 kernel")


def test_sum_norm_oracle_reproduces_the_reference_kernel(q27, orc):
    """The reference's sum_norm_q8 kernel (no exchange) on a B200, from tests/golden/make_golden_sum_norm.py:
    the sum is exact, the normalised row agrees to the last bits (the block sum's tree and the fast-math
    rsqrt are the reference's), and q8_1 of the reference's own row gives its bytes and scales."""
    from golden_cases import SUM_NORM_EPS, sum_norm_inputs
    g = np.load(os.path.join(ROOT, "tests", "golden", "ref_sum_norm_b200.npz"))
    x, part, w = sum_norm_inputs()
    xn, h = orc.sum_norm(x, [part], w, SUM_NORM_EPS)
    assert np.array_equal(xn, g["x"])
    np.testing.assert_allclose(h, g["h"], rtol=2e-6, atol=1e-7)
    rq, rd = orc.q8_1(g["h"].reshape(-1))
    off = rq.astype(np.int32) - g["xq"].reshape(-1).astype(np.int32)
    assert np.abs(off).max() <= 1 and (off != 0).mean() <= 1e-4  # the reference divides with fast-math
    assert np.array_equal(rd, g["xd"])


# ---------------------------------------------------------------- cases at depth (ref_b200_deep.npz)
DEEP_PATH = os.path.join(ROOT, "tests", "golden", "ref_b200_deep.npz")


@pytest.fixture(scope="module")
def deep():
    assert os.path.exists(DEEP_PATH), "deep fixture missing: run tests/golden/make_golden.py --deep on a B200"
    return np.load(DEEP_PATH)


def _q8_rows_close(vals, sc, ref_vals, ref_sc, what, frac=2e-3):
    """q8_0 rows against the reference kernel's: the reference divides with fast-math, so a value on a
    rounding boundary may sit one step off and a scale one f16 ulp off; nothing else may differ."""
    d = np.abs(vals.astype(np.int32) - ref_vals.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() <= frac, "%s: max step %d, %.2e of values differ" % (what, d.max(), (d != 0).mean())
    a, b = sc.astype(np.float32), ref_sc.astype(np.float32)
    assert (np.abs(a - b) <= np.abs(b) * 2.0 ** -10 + 1e-12).all(), "%s: scales differ" % what


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["prep_q8", "prep_f16", "prep_q8_many", "prep_q8_deep", "prep_q8_rope3"])
def test_attn_prep_kernel_against_reference_kernel(gold, deep, q27, name):
    """q27b_attn_prep (RMSNorm + IMRoPE + cache write) against the outputs of the reference's own
    attn_prep kernel on the same seeded inputs: the query rows, and the K and V cache rows it wrote.
    Both builds use the fast sine / cosine / power instructions, so the rotation agrees to rounding
    even where the angle is ~1.5e5 rad (position 150,000)."""
    import torch
    from golden_cases import CASES_ALL, DEEP_CASES
    from helpers_gpu import dev, pos_tensor
    c = CASES_ALL[name]
    g = deep if name in DEEP_CASES else gold
    x = case_inputs(name)
    T, nqh, nkvh, n_ctx, pos0, q8 = c["T"], c["nqh"], c["nkvh"], c["n_ctx"], c["pos0"], c["q8"]
    qn = torch.full((T, nqh, AD), float("nan"), device="cuda")
    kc, vc = q27.new_cache(nkvh, n_ctx, q8), q27.new_cache(nkvh, n_ctx, q8)
    rope3 = dev(np.array(c["rope3"], np.int32)) if c.get("rope3") else None
    q27.attn_prep(dev(x["qg"]), dev(x["k"]), dev(x["v"]), dev(x["q_norm"]), dev(x["k_norm"]), qn, kc, vc,
                  pos_tensor(pos0), T, c["eps"], c["theta_scale"], nqh, nkvh, n_ctx, q8, rope3=rope3)
    torch.cuda.synchronize()
    assert q27.device_status() == 0
    if name + "/qn" in g.files:
        ref = g[name + "/qn"]
        got = qn.cpu().numpy()
        # RMSNorm sums in a different order; the rotation uses the same approximate instructions
        assert np.abs(got - ref).max() <= 2e-5 * max(1.0, float(np.abs(ref).max())), \
            "%s qn: max diff %.3e" % (name, np.abs(got - ref).max())
    if not q8:
        kr = g[name + "/kcache"].view(np.float16).astype(np.float32)
        kg = kc.cpu().numpy().view(np.float16).astype(np.float32)
        assert np.abs(kg - kr).max() <= 2e-3 * max(1.0, float(np.abs(kr).max()))  # one f16 step of the largest value
        assert np.array_equal(vc.cpu().numpy(), g[name + "/vcache"])
        return
    for key, cache in (("k", kc), ("v", vc)):
        got = cache.cpu().numpy()
        vals = got[: nkvh * n_ctx * AD].view(np.int8).reshape(nkvh, n_ctx, AD)
        sc = got[nkvh * n_ctx * AD:].view(np.float16).reshape(nkvh, n_ctx, 8)
        if c.get("rows_only"):
            rv, rs = g[name + "/%srows" % key].view(np.int8), g[name + "/%sscales" % key]
            _q8_rows_close(vals[:, pos0:pos0 + T], sc[:, pos0:pos0 + T], rv, rs, "%s %s rows" % (name, key))
            untouched = np.ones(n_ctx, bool)
            untouched[pos0:pos0 + T] = False
            assert (vals[:, untouched] == 0).all()
        else:
            rv, rs = split_q8(g[name + "/%scache" % key], nkvh, n_ctx)
            _q8_rows_close(vals, sc, rv, rs, "%s %s cache" % (name, key))


def test_decode_oracle_at_depth_against_reference_kernels(deep, orc):
    from golden_cases import DEEP_CASES
    c = DEEP_CASES["decode_deep"]
    x = case_inputs("decode_deep")
    kc, vc = orc.fill_cache(x["k"], x["v"], c["n_ctx"], c["q8"])
    o = orc.attn_ref(x["qn"], x["qg"], kc, vc, c["n"] - c["T"], c["scale"], c["nkvh"], c["n_ctx"], c["q8"])
    assert_close(o, deep["decode_deep/slow"], "decode_deep vs attn_decode_ref", abs_tol=5e-5, rel_tol=2e-3)
    assert_close(o, deep["decode_deep/fast"], "decode_deep vs attn_decode")


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", [1, 2, 3, 4], ids=["mma", "tc", "ws", "wt"])
def test_new_decode_kernels_at_depth_against_reference_outputs(deep, q27, orc, kernel):
    """40,000 positions: every split-K kernel of the library against what the reference's slow and fast
    decode kernels gave for the same seeded inputs."""
    import torch
    from golden_cases import DEEP_CASES
    from helpers_gpu import dev, pos_tensor
    c = DEEP_CASES["decode_deep"]
    x = case_inputs("decode_deep")
    nqh = c["nkvh"] * 6
    kc, vc = orc.fill_cache(x["k"], x["v"], c["n_ctx"], True)
    o = torch.empty((c["T"], nqh, AD), device="cuda")
    q27.set_decode_kernel(kernel)
    try:
        q27.attn_decode(dev(x["qn"]), dev(x["qg"]), dev(kc), dev(vc), o, None, None, pos_tensor(c["n"] - c["T"]), c["T"],
                        c["scale"], nqh, c["nkvh"], c["n_ctx"])
        torch.cuda.synchronize()
    finally:
        q27.set_decode_kernel(0)
    assert_close(o.cpu().numpy(), deep["decode_deep/slow"], "new kernel vs the reference's slow kernel at 40k")
    assert_close(o.cpu().numpy(), deep["decode_deep/fast"], "new kernel vs the reference's fast kernel at 40k")
    assert q27.device_status() == 0


def _close_to_f16_accumulating_kernel(a, ref, what):
    """The reference's prefill kernel keeps its O accumulators in f16 (src/attn.cu:321,736,776-785), so its own
    error grows with the depth (at 8,192 positions single values are off by 3 % of the output RMS against
    an f32 accumulation). Against it the path's tolerance is taken as stated: max-abs <= 2e-3 and relative
    L2 <= 1e-2, without the per-value bound relative to the RMS that the other comparisons add."""
    mx, rms, l2 = err_stats(a, ref)
    assert np.isfinite(np.asarray(a)).all() and mx <= 2e-3 and l2 <= 1e-2, \
        "%s: max err %.3e, ref rms %.3e, rel L2 %.3e" % (what, mx, rms, l2)


def test_prefill_oracle_at_depth_against_reference_kernel(deep, orc):
    from golden_cases import DEEP_CASES
    c = DEEP_CASES["prefill_deep"]
    x = case_inputs("prefill_deep")
    kc, vc = orc.fill_cache(x["k"], x["v"], c["n_ctx"], True)
    for a, b in c["keep"]:
        o = orc.attn_prefill_i8(x["qn"], x["qg"], kc, vc, c["pos0"], c["scale"], c["nkvh"], c["n_ctx"], a, b)[a:b]
        _close_to_f16_accumulating_kernel(o, deep["prefill_deep/i8_%d_%d" % (a, b)],
                                          "prefill_deep tokens %d..%d vs attn_prefill (int8)" % (a, b))


@pytest.mark.gpu
@pytest.mark.parametrize("kernel", [1, 2], ids=["int8", "f16qk"])
def test_new_prefill_kernels_at_depth_against_reference_outputs(deep, q27, orc, kernel):
    """256 tokens on an 8,192-token prefix: both prefill kernels against the reference's int8 kernel
    (sampled token ranges; the f16-QK route differs from it by the int8 rounding of Q only)."""
    import torch
    from golden_cases import DEEP_CASES
    from helpers_gpu import dev, pos_tensor
    c = DEEP_CASES["prefill_deep"]
    x = case_inputs("prefill_deep")
    nqh = c["nkvh"] * 6
    kc, vc = orc.fill_cache(x["k"], x["v"], c["n_ctx"], True)
    o = torch.empty((c["M"], nqh, AD), device="cuda")
    q27.set_prefill_kernel(kernel)
    try:
        q27.attn_prefill(dev(x["qn"]), dev(x["qg"]), dev(kc), dev(vc), o, pos_tensor(c["pos0"]), c["M"], c["scale"], nqh,
                         c["nkvh"], c["n_ctx"], True, c["pos0"])
        torch.cuda.synchronize()
    finally:
        q27.set_prefill_kernel(0)
    got = o.cpu().numpy()
    for a, b in c["keep"]:
        ref = deep["prefill_deep/i8_%d_%d" % (a, b)]
        if kernel == 1:
            _close_to_f16_accumulating_kernel(got[a:b], ref, "int8 prefill at depth, tokens %d..%d" % (a, b))
        else:
            assert_close(got[a:b], ref, "f16-QK prefill at depth, tokens %d..%d" % (a, b), abs_tol=5e-3, rel_tol=5e-2)
    assert q27.device_status() == 0
