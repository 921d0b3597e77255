"""The seeded cases of tests/golden/ref_b200.npz, shared by the script that makes the fixture (on
a B200, from the reference's own kernels) and the tests that read it."""
import numpy as np

AD = 256

CASES = {
    # attn_prep: RMSNorm + RoPE + cache write. The V rows pin the q8_0 quantiser (V is written raw).
    "prep_q8": dict(kind="prep", T=4, nqh=12, nkvh=2, n_ctx=64, pos0=20, q8=True, eps=1e-6,
                    theta_scale=float(10000000.0 ** (-2.0 / 64))),
    "prep_f16": dict(kind="prep", T=2, nqh=6, nkvh=1, n_ctx=16, pos0=3, q8=False, eps=1e-6,
                     theta_scale=float(10000000.0 ** (-2.0 / 64))),
    "prep_q8_many": dict(kind="prep", T=256, nqh=6, nkvh=1, n_ctx=256, pos0=0, q8=True, eps=1e-6,
                         theta_scale=float(10000000.0 ** (-2.0 / 64))),
    # decode: the reference's slow kernel (attn_decode_ref) and its fast kernel (attn_decode)
    "decode_cfg1": dict(kind="decode", T=1, nkvh=4, n=1024, n_ctx=1024, q8=True, scale=1 / 16),
    "decode_t4": dict(kind="decode", T=4, nkvh=2, n=2500, n_ctx=2504, q8=True, scale=1 / 16, q8_1=True),
    "decode_f16": dict(kind="decode", T=4, nkvh=1, n=700, n_ctx=704, q8=False, scale=1 / 16),
    # prefill: the reference's int8 Q K^T kernel, and its slow f16-Q kernel on the same rows
    "prefill_a": dict(kind="prefill", M=24, nkvh=1, pos0=300, n_ctx=328, scale=1 / 16),
    "prefill_b": dict(kind="prefill", M=17, nkvh=1, pos0=0, n_ctx=20, scale=1 / 16),
}


# Cases at depth, in a fixture of their own (tests/golden/ref_b200_deep.npz), which keeps only what the
# tests compare: query rows and the cache rows just written (prep), the output (decode), sampled token
# ranges of the output (prefill). Inputs are regenerated from the seeds.
DEEP_CASES = {
    # attn_prep at the depth the metric is quoted at: the rotation angle of dim 0 is ~1.5e5 rad, where the
    # fast sine / cosine of the reference's build (-use_fast_math) are far from the exact ones
    "prep_q8_deep": dict(kind="prep", T=4, nqh=12, nkvh=2, n_ctx=150016, pos0=150000, q8=True, eps=1e-6,
                         theta_scale=float(10000000.0 ** (-2.0 / 64)), rows_only=True),
    # IMRoPE sections with large time / height / width positions
    "prep_q8_rope3": dict(kind="prep", T=4, nqh=12, nkvh=2, n_ctx=64, pos0=20, q8=True, eps=1e-6,
                          theta_scale=float(10000000.0 ** (-2.0 / 64)), rows_only=True,
                          rope3=[[120000, 300, 77], [120001, 300, 78], [120002, 301, 77], [149999, 2047, 2047]]),
    "decode_deep": dict(kind="decode", T=4, nkvh=2, n=40000, n_ctx=40000, q8=True, scale=1 / 16),
    "prefill_deep": dict(kind="prefill", M=256, nkvh=1, pos0=8192, n_ctx=8448, scale=1 / 16,
                         keep=[(0, 8), (124, 132), (248, 256)]),
}
CASES_ALL = dict(CASES, **DEEP_CASES)


def case_inputs(name):
    from qwen27_engine_b200 import synth
    c = CASES_ALL[name]
    # disjoint slices of the streams per case
    tag = (sorted(CASES).index(name) + 1 if name in CASES else 17 + sorted(DEEP_CASES).index(name)) << 26
    if c["kind"] == "prep":
        T, nqh, nkvh = c["T"], c["nqh"], c["nkvh"]
        return dict(qg=synth.normal(synth.SEED_Q, (T, nqh, 512), start=tag),
                    k=synth.normal(synth.SEED_K, (T, nkvh, AD), start=tag),
                    v=synth.normal(synth.SEED_V, (T, nkvh, AD), start=tag) * np.float32(1.7),
                    q_norm=(1 + 0.1 * synth.normal(synth.SEED_GATE, (AD,), start=tag)).astype(np.float32),
                    k_norm=(1 + 0.1 * synth.normal(synth.SEED_GATE, (AD,), start=tag + 4096)).astype(np.float32))
    if c["kind"] == "decode":
        T, nkvh, n = c["T"], c["nkvh"], c["n"]
        nqh = nkvh * 6
        qn = synth.normal(synth.SEED_Q, (T, nqh, AD), start=tag)
        qg = np.zeros((T, nqh, 512), np.float32)
        qg[..., 256:] = synth.normal(synth.SEED_GATE, (T, nqh, AD), start=tag)
        return dict(qn=qn, qg=qg, k=synth.normal(synth.SEED_K, (nkvh, n, AD), start=tag),
                    v=synth.normal(synth.SEED_V, (nkvh, n, AD), start=tag))
    M, nkvh, n = c["M"], c["nkvh"], c["pos0"] + c["M"]
    nqh = nkvh * 6
    qn = synth.normal(synth.SEED_Q, (M, nqh, AD), start=tag)
    qg = np.zeros((M, nqh, 512), np.float32)
    qg[..., 256:] = synth.normal(synth.SEED_GATE, (M, nqh, AD), start=tag)
    return dict(qn=qn, qg=qg, k=synth.normal(synth.SEED_K, (nkvh, n, AD), start=tag),
                v=synth.normal(synth.SEED_V, (nkvh, n, AD), start=tag))


SUM_NORM_EPS = 1e-6


def sum_norm_inputs():
    """x [4][5120], partial [4][5120], w [5120] of the sum_norm_q8 fixture (the reference's kernel takes n = 5120 only)."""
    from qwen27_engine_b200 import synth
    rows, n = 4, 5120
    x = synth.normal(synth.SEED_Q, (rows, n), start=7 << 20)
    part = (0.3 * synth.normal(synth.SEED_K, (rows, n), start=7 << 20)).astype(np.float32)
    w = (1.0 + 0.1 * synth.normal(synth.SEED_GATE, (n,), start=7 << 20)).astype(np.float32)
    return x, part, w
