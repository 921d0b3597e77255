"""The drop-in boundary on the GPU: the reference's own check-and-bench tool running on the new kernels
through the shim headers, the tensor-map cache under more caches than the reference engine holds, and
the workspace that never moves after warm-up."""
import os
import re
import subprocess

import numpy as np
import pytest
import torch

from conftest import ROOT, assert_close
from helpers_gpu import dev, pos_tensor

pytestmark = pytest.mark.gpu
AD, GQA = 256, 6
SCALE = 1.0 / 16.0


def _run_tool(exe):
    r = subprocess.run([exe, "0", "30000", "q8"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    pf = re.findall(r"prefill pos0\s+(\d+) M\s+(\d+):.*max err ([0-9.e+-]+) \(ref rms ([0-9.]+)\)", r.stdout)
    dc = re.findall(r"depth\s+(\d+) T=(\d):.*max err ([0-9.e+-]+) \(ref rms ([0-9.]+)\)", r.stdout)
    assert len(pf) == 4 and len(dc) == 14, r.stdout  # the tool's cases up to 30,000 positions
    return {(a, b): (float(e), float(rms)) for a, b, e, rms in pf}, {(a, b): (float(e), float(rms)) for a, b, e, rms in dc}


def test_reference_bench_tool_on_the_new_kernels():
    """tools/bench_attn.cu of the reference, compiled unmodified against qwen27-engine_b200/shim and linked
    with libq27b_attn.so (oracle/build.py: build_bench_attn), run as it is: it compares attn_prefill and
    attn_decode with attn_decode_ref on its own xorshift data (2 KV heads, 12 Q heads, q8_0; Q uniform in
    +-2.5, K and V bytes uniform over the whole int8 range) and prints `max err` and `ref rms` per case,
    without a threshold of its own. Every decode case must be within the path's tolerance. The prefill
    cases compare int8-rounded Q with the f16-Q definition on data where that rounding alone moves single
    values by several per cent of the RMS: there the bar is what the same tool prints for the reference's
    own kernels on this GPU (oracle/_ref/bench_attn_ref), which the new kernel must not exceed."""
    exe = os.path.join(ROOT, "oracle", "_ref", "bench_attn_shim")
    ref_exe = os.path.join(ROOT, "oracle", "_ref", "bench_attn_ref")
    if not os.path.exists(exe) or not os.path.exists(ref_exe):
        pytest.skip("oracle/_ref/bench_attn_shim / bench_attn_ref are not built (they need the reference checkout at build time)")
    pf, dc = _run_tool(exe)
    rpf, rdc = _run_tool(ref_exe)
    for key, (err, rms) in dc.items():
        assert err <= 2e-3 and err <= 1e-2 * rms, "decode depth %s T %s: %g (rms %g)" % (key + (err, rms))
        assert abs(rms - rdc[key][1]) <= 2e-3 * max(rms, 1e-3) + 1e-3  # the same problem in both programs
    for key, (err, rms) in pf.items():
        assert err <= 1.25 * rpf[key][0] + 1e-4, "prefill pos0 %s M %s: max err %g, the reference's kernel has %g (rms %g)" % (
            key + (err, rpf[key][0], rms))


def test_seventy_caches_through_decode_and_prefill(q27, orc):
    """The reference engine keeps 17 layers x (K, V) x 2 cards = 68 caches alive in one process
    (src/model.cu:462-472); 70 distinct cache pairs go through decode and prefill twice here (the second
    round finds every tensor map in the cache) and every result is checked."""
    from qwen27_engine_b200 import synth
    nkvh, T, n, M = 1, 4, 200, 16
    nqh, n_ctx = nkvh * GQA, 224
    qn = synth.normal(synth.SEED_Q, (M, nqh, AD))
    qg = np.zeros((M, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (M, nqh, AD))
    dq, dg = dev(qn), dev(qg)
    cases = []
    for i in range(70):
        kf = synth.normal(synth.SEED_K, (nkvh, n, AD), start=i << 20)
        vf = synth.normal(synth.SEED_V, (nkvh, n, AD), start=i << 20)
        kc, vc = orc.fill_cache(kf, vf, n_ctx)
        ref_d = orc.attn_ref(qn[:T], qg[:T], kc, vc, n - T, SCALE, nkvh, n_ctx)
        ref_p = orc.attn_prefill_i8(qn, qg, kc, vc, n - M, SCALE, nkvh, n_ctx)
        cases.append((dev(kc), dev(vc), ref_d, ref_p))
    od = torch.empty((T, nqh, AD), device="cuda")
    op = torch.empty((M, nqh, AD), device="cuda")
    for rnd in range(2):
        for i, (kc, vc, ref_d, ref_p) in enumerate(cases):
            q27.attn_decode(dq[:T].contiguous(), dg[:T].contiguous(), kc, vc, od, None, None, pos_tensor(n - T), T, SCALE,
                            nqh, nkvh, n_ctx)
            q27.attn_prefill(dq, dg, kc, vc, op, pos_tensor(n - M), M, SCALE, nqh, nkvh, n_ctx)
            torch.cuda.synchronize()
            assert_close(od.cpu().numpy(), ref_d, "decode, cache %d, round %d" % (i, rnd))
            assert_close(op.cpu().numpy(), ref_p, "prefill, cache %d, round %d" % (i, rnd))
    assert q27.device_status() == 0


def test_workspace_does_not_move_after_warm_up(q27, orc):
    """A deeper prefill after warm-up must not free or grow anything: the workspace sizes stay what the
    first calls made them, and a decode graph captured before still replays correctly afterwards
    (the reference fixes its prefill buffer for the same reason, src/attn.cu:954-959)."""
    from qwen27_engine_b200 import synth
    nkvh, T, n = 2, 4, 20000
    nqh, n_ctx = nkvh * GQA, n + 8
    qn, qg, kf, vf = synth.decode_inputs(T, nqh, nkvh, n)
    kc_ref, vc_ref = orc.fill_cache(kf, vf, n_ctx)
    kc, vc, dq, dg = dev(kc_ref), dev(vc_ref), dev(qn), dev(qg)
    o = torch.empty((T, nqh, AD), device="cuda")
    pos = pos_tensor(n - T)
    q27.attn_decode(dq, dg, kc, vc, o, None, None, pos, T, SCALE, nqh, nkvh, n_ctx)
    M = 256
    pqn = torch.randn((M, nqh, AD), device="cuda")
    pqg = torch.randn((M, nqh, 512), device="cuda")
    po = torch.empty((M, nqh, AD), device="cuda")
    q27.attn_prefill(pqn, pqg, kc, vc, po, pos_tensor(4096), M, SCALE, nqh, nkvh, n_ctx, True, 4096)  # shallow: two pieces
    torch.cuda.synchronize()
    before = q27.workspace_query()
    assert before[0] > 0 and before[1] > 0
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        q27.attn_decode(dq, dg, kc, vc, o, None, None, pos, T, SCALE, nqh, nkvh, n_ctx)
    free0 = torch.cuda.mem_get_info()[0]
    q27.attn_prefill(pqn, pqg, kc, vc, po, pos_tensor(n - M), M, SCALE, nqh, nkvh, n_ctx, True, n - M)  # deep: more pieces
    torch.cuda.synchronize()
    assert q27.workspace_query() == before
    assert torch.cuda.mem_get_info()[0] == free0
    o.fill_(float("nan"))
    g.replay()
    torch.cuda.synchronize()
    assert_close(o.cpu().numpy(), orc.attn_ref(qn, qg, kc_ref, vc_ref, n - T, SCALE, nkvh, n_ctx), "replayed decode graph")
    assert q27.device_status() == 0


def test_fixed_workspace_refuses_to_grow(q27):
    """After q27b_attn_workspace_init nothing is allocated any more: a paged decode that needs more than
    it was given fails with a message that names both sizes; destroy lifts the fix."""
    q27.workspace_destroy()
    q27.workspace_init(16 << 20, 1 << 20)
    try:
        d, p, g, fixed = q27.workspace_query()
        assert fixed and p == 16 << 20 and g == 1 << 20 and d > 0
        nkvh, nqh, T, B, n = 2, 12, 4, 8, 3000
        n_pages = 8 * 12 + 1
        pool = torch.zeros(q27.kv_pool_bytes(nkvh, n_pages), dtype=torch.uint8, device="cuda")
        tables = torch.arange(B * 12, dtype=torch.int32, device="cuda").view(B, 12)
        lens = torch.full((B,), n, dtype=torch.int32, device="cuda")
        o = torch.empty((B, T, nqh, AD), device="cuda")
        with pytest.raises(q27.Q27Error) as e:
            q27.attn_decode_paged(torch.zeros((B, T, nqh, AD), device="cuda"), torch.zeros((B, T, nqh, 512), device="cuda"),
                                  pool, pool, tables, lens, o, B, T, SCALE, nqh, nkvh, n_pages, 12, n)
        assert e.value.code == q27.UNSUPPORTED and "workspace" in str(e.value)
        assert q27.workspace_query() == (d, p, g, True)
    finally:
        q27.workspace_destroy()
    assert q27.workspace_query() == (0, 0, 0, False)
