"""KV append / q8_0 quantise and the attn_prep prologue on the GPU, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from helpers_gpu import dev, pos_tensor

pytestmark = pytest.mark.gpu
AD = 256


@pytest.mark.parametrize("q8", [True, False])
@pytest.mark.parametrize("T,pos0", [(1, 0), (4, 61), (3, 1000), (100, 7)])
def test_kv_append_bit_exact(q27, orc, q8, T, pos0):
    rng = np.random.default_rng(T * 1000 + pos0)
    nkvh, n_ctx = 4, pos0 + T + 5
    k = rng.standard_normal((T, nkvh, AD)).astype(np.float32)
    v = (rng.standard_normal((T, nkvh, AD)) * 3).astype(np.float32)
    k[0, 0, :32] = 0           # an all-zero block: scale 0, values 0
    v[0, 1, 5] = 1e-30         # tiny values
    if T > 2:
        k[2, 0] = 0.5          # ties at .5 after scaling: roundf goes away from zero
    kc_ref, vc_ref = orc.new_cache(nkvh, n_ctx, q8, fill=0xAB), orc.new_cache(nkvh, n_ctx, q8, fill=0xAB)
    orc.kv_append(k, v, kc_ref, vc_ref, pos0, nkvh, n_ctx, q8)
    kc, vc = q27.new_cache(nkvh, n_ctx, q8, fill=0xAB), q27.new_cache(nkvh, n_ctx, q8, fill=0xAB)
    q27.kv_append(dev(k), dev(v), kc, vc, pos_tensor(pos0), T, nkvh, n_ctx, q8)
    torch.cuda.synchronize()
    # every byte, including the 0xAB canaries of the rows that must stay untouched
    assert np.array_equal(kc.cpu().numpy(), kc_ref)
    assert np.array_equal(vc.cpu().numpy(), vc_ref)
    assert q27.device_status() == 0


def test_kv_append_never_writes_outside(q27):
    nkvh, n_ctx, T = 2, 8, 4
    kc, vc = q27.new_cache(nkvh, n_ctx, True, fill=0xCD), q27.new_cache(nkvh, n_ctx, True, fill=0xCD)
    k = torch.ones((T, nkvh, AD), device="cuda")
    q27.kv_append(k, k, kc, vc, pos_tensor(6), T, nkvh, n_ctx, True)  # rows 8, 9 do not exist
    torch.cuda.synchronize()
    vals = kc[: nkvh * n_ctx * AD].view(nkvh, n_ctx, AD).cpu().numpy()
    assert (vals[:, :6] == 0xCD).all() and (vals[:, 6:8] == 127).all()


def np_prep(qg, k, q_norm, k_norm, pos, eps, theta_scale, rope3=None):
    """attn_prep's norm + NeoX RoPE on dims 0..63 (reference src/ops.cu:609-627), in float64."""
    def one(x, w, tok):
        x = x.astype(np.float64)
        y = x / np.sqrt((x * x).mean() + eps) * w
        out = y.copy()
        for j in range(32):
            rp = rope3[tok][j % 3] if rope3 is not None else pos[tok]
            th = rp * theta_scale ** j
            c, s = np.cos(th), np.sin(th)
            out[j] = y[j] * c - y[j + 32] * s
            out[j + 32] = y[j] * s + y[j + 32] * c
        return out
    T, nqh = qg.shape[:2]
    qn = np.stack([[one(qg[t, h, :256], q_norm, t) for h in range(nqh)] for t in range(T)])
    kn = np.stack([[one(k[t, h], k_norm, t) for h in range(k.shape[1])] for t in range(T)])
    return qn, kn


@pytest.mark.parametrize("use_rope3", [False, True])
def test_attn_prep(q27, orc, use_rope3):
    rng = np.random.default_rng(11)
    T, nqh, nkvh, n_ctx, pos0 = 4, 12, 2, 64, 20
    qg = rng.standard_normal((T, nqh, 512)).astype(np.float32)
    k = rng.standard_normal((T, nkvh, AD)).astype(np.float32)
    v = rng.standard_normal((T, nkvh, AD)).astype(np.float32)
    qw = (1 + 0.1 * rng.standard_normal(AD)).astype(np.float32)
    kw = (1 + 0.1 * rng.standard_normal(AD)).astype(np.float32)
    eps, theta_scale = 1e-6, float(10000000.0 ** (-2.0 / 64))
    rope3 = rng.integers(0, 40, (T, 3)).astype(np.int32) if use_rope3 else None
    rdelta = None if use_rope3 else 3
    pos = [pos0 + t - (rdelta or 0) for t in range(T)]
    qn_ref, kn_ref = np_prep(qg, k, qw, kw, pos, eps, theta_scale, rope3)
    qn = torch.empty((T, nqh, AD), device="cuda")
    kc, vc = q27.new_cache(nkvh, n_ctx), q27.new_cache(nkvh, n_ctx)
    q27.attn_prep(dev(qg), dev(k), dev(v), dev(qw), dev(kw), qn, kc, vc, pos_tensor(pos0), T, eps, theta_scale, nqh,
                  nkvh, n_ctx, True, rope3=dev(rope3) if use_rope3 else None,
                  rdelta=None if use_rope3 else pos_tensor(rdelta))
    torch.cuda.synchronize()
    assert np.abs(qn.cpu().numpy() - qn_ref).max() < 2e-5
    # V rows are quantised raw: bit-exact; K rows are the quantised normed + roped rows
    kc_ref, vc_ref = orc.new_cache(nkvh, n_ctx), orc.new_cache(nkvh, n_ctx)
    orc.kv_append(kn_ref.astype(np.float32), v, kc_ref, vc_ref, pos0, nkvh, n_ctx)
    assert np.array_equal(vc.cpu().numpy(), vc_ref)
    got = kc.cpu().numpy()
    vals, ref_vals = got[: nkvh * n_ctx * AD].view(np.int8), kc_ref[: nkvh * n_ctx * AD].view(np.int8)
    diff = np.abs(vals.astype(np.int32) - ref_vals.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3  # f32 vs f64 norm: a few values on a rounding boundary
    f16 = lambda a: a[nkvh * n_ctx * AD:].view(np.float16).astype(np.float32)
    assert np.abs(f16(got) - f16(kc_ref)).max() <= 2e-5
