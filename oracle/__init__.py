"""ctypes bindings of the CPU oracle (oracle/attn_oracle.cpp) on numpy arrays.

Test infrastructure only: imported by tests/, the smoke check and the cpu_baseline leg of the
benchmark. The shipped package never imports this module.
"""
import ctypes
import os

import numpy as np

from . import build as _build

AD = 256
GQA = 6
PROW = AD + 2

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO
        if not os.path.exists(path):
            path = _build.build_oracle()
        _lib = ctypes.CDLL(path)
        _lib.orc_kv_cache_bytes.restype = ctypes.c_uint64
    return _lib


def _p(a):
    return ctypes.c_void_p(a.ctypes.data) if a is not None else ctypes.c_void_p(0)


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


def num_threads():
    return int(lib().orc_num_threads())


def kv_cache_bytes(nkvh, n_ctx, q8=True):
    return int(lib().orc_kv_cache_bytes(nkvh, n_ctx, int(q8)))


def quant_q8_0(x):
    """x [..., 256] f32 -> (int8 [..., 256], f16-bit scales uint16 [..., 8])."""
    x = _c(x, np.float32)
    rows = x.size // AD
    q = np.empty(x.shape, np.int8)
    d = np.empty(x.shape[:-1] + (8,), np.uint16)
    lib().orc_quant_q8_0(_p(x), ctypes.c_int64(rows), _p(q), _p(d))
    return q, d


def new_cache(nkvh, n_ctx, q8=True, fill=0):
    return np.full(kv_cache_bytes(nkvh, n_ctx, q8), fill, np.uint8)


def kv_append(k, v, kcache, vcache, pos0, nkvh, n_ctx, q8=True):
    """k, v [T][nkvh][256] f32 written in place at cache rows pos0 + t."""
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    T = k.shape[0]
    assert pos0 >= 0 and pos0 + T <= n_ctx
    lib().orc_kv_append(_p(k), _p(v), _p(kcache), _p(vcache), int(pos0), int(T), int(nkvh), int(n_ctx), int(q8))


def fill_cache(kf, vf, n_ctx, q8=True):
    """kf, vf [nkvh][n][256] f32 -> (kcache, vcache) byte arrays with rows 0..n-1 filled."""
    nkvh, n = kf.shape[0], kf.shape[1]
    kc, vc = new_cache(nkvh, n_ctx, q8), new_cache(nkvh, n_ctx, q8)
    for src, c in ((kf, kc), (vf, vc)):
        if q8:
            q, d = quant_q8_0(src)
            c[: nkvh * n_ctx * AD].reshape(nkvh, n_ctx, AD)[:, :n] = q.view(np.uint8)
            c[nkvh * n_ctx * AD:].view(np.uint16).reshape(nkvh, n_ctx, 8)[:, :n] = d
        else:
            c.view(np.float16).reshape(nkvh, n_ctx, AD)[:, :n] = src.astype(np.float16)
    return kc, vc


def q8_1(y):
    y = _c(y, np.float32)
    xq = np.empty(y.shape, np.int8)
    xd = np.empty(y.size // 32, np.float32)
    lib().orc_q8_1(_p(y), ctypes.c_int64(y.size), _p(xq), _p(xd))
    return xq, xd


def sum_norm(x, partials, w, eps):
    """The reference's sum_norm_q8 (src/ops.cu:129-260, non-exchange branch, and norm_q8_row :89-107) for
    a list of per-rank partials: x_new = x + (p0 + p1 + ..) in f32 in rank order, scale =
    1 / sqrt(mean(x_new^2) + eps) with the mean taken in f64 (the kernel's f32 tree may differ in the last
    bit), h = scale * x_new * w in f32. Returns (x_new, h); the q8_1 form is q8_1(h)."""
    x = _c(x, np.float32)
    s = _c(partials[0], np.float32).copy()
    for p in partials[1:]:
        s = s + _c(p, np.float32)
    xn = x + s
    t = (xn.astype(np.float64) ** 2).sum(axis=-1, keepdims=True)
    scale = (1.0 / np.sqrt(t / xn.shape[-1] + np.float64(np.float32(eps)))).astype(np.float32)
    h = (scale * xn) * _c(w, np.float32)
    return xn, h.astype(np.float32)


def attn_ref(qn, qg, kcache, vcache, pos0, kq_scale, nkvh, n_ctx, q8=True):
    """qn [T][nqh][256], qg [T][nqh][512] -> o [T][nqh][256] (decode numerics)."""
    qn = _c(qn, np.float32)
    qg = _c(qg, np.float32)
    T, nqh = qn.shape[0], qn.shape[1]
    assert nqh == nkvh * GQA and pos0 + T <= n_ctx
    o = np.empty((T, nqh, AD), np.float32)
    lib().orc_attn_ref(_p(qn), _p(qg), _p(kcache), _p(vcache), _p(o), int(pos0), int(T), ctypes.c_float(kq_scale),
                       int(nqh), int(nkvh), int(n_ctx), int(q8))
    return o


def attn_partial(qn, kcache, vcache, pos0, kq_scale, nkvh, n_ctx, p_lo, p_hi, q8=True):
    """(m, l, O) partial [T][nqh][258] over positions [p_lo, p_hi)."""
    qn = _c(qn, np.float32)
    T, nqh = qn.shape[0], qn.shape[1]
    part = np.zeros((T, nqh, PROW), np.float32)
    lib().orc_attn_partial(_p(qn), _p(kcache), _p(vcache), _p(part), int(pos0), int(T), ctypes.c_float(kq_scale),
                           int(nqh), int(nkvh), int(n_ctx), int(q8), int(p_lo), int(p_hi))
    return part


def lse_merge(parts, qg=None):
    """parts [nparts][rows...][258]; qg [rows...][512] or None -> o [rows...][256]."""
    parts = _c(parts, np.float32)
    nparts = parts.shape[0]
    rows = parts[0].size // PROW
    o = np.empty(parts.shape[1:-1] + (AD,), np.float32)
    g = _c(qg, np.float32) if qg is not None else None
    lib().orc_lse_merge(_p(parts), int(nparts), ctypes.c_int64(rows * PROW), ctypes.c_int64(rows), _p(g), _p(o))
    return o


def quant_q_i8(x, kq_scale):
    x = _c(x, np.float32)
    q = np.empty(x.shape, np.int8)
    d = np.empty(x.shape[:-1] + (8,), np.float32)
    lib().orc_quant_q_i8(_p(x), ctypes.c_int64(x.size // AD), ctypes.c_float(kq_scale), _p(q), _p(d))
    return q, d


def qk_i32(q, k):
    """q [rows][256] int8, k [npos][256] int8 -> int32 [rows][npos][8] block dot products."""
    q = _c(q, np.int8)
    k = _c(k, np.int8)
    out = np.empty((q.shape[0], k.shape[0], 8), np.int32)
    lib().orc_qk_i32(_p(q), _p(k), int(q.shape[0]), int(k.shape[0]), _p(out))
    return out


def attn_prefill_i8(qn, qg, kcache, vcache, pos0, kq_scale, nkvh, n_ctx, t_lo=0, t_hi=None):
    """qn [M][nqh][256], qg [M][nqh][512] -> o [M][nqh][256]; only tokens [t_lo, t_hi) are filled."""
    qn = _c(qn, np.float32)
    qg = _c(qg, np.float32)
    M, nqh = qn.shape[0], qn.shape[1]
    t_hi = M if t_hi is None else t_hi
    o = np.zeros((M, nqh, AD), np.float32)
    lib().orc_attn_prefill_i8(_p(qn), _p(qg), _p(kcache), _p(vcache), _p(o), int(pos0), int(M),
                              ctypes.c_float(kq_scale), int(nqh), int(nkvh), int(n_ctx), int(t_lo), int(t_hi))
    return o


def kv_wire_from_cache(cache, nkvh, n_ctx, p0, p1):
    """Rows [p0, p1) of a contiguous q8_0 cache in the reference's host layout: the values
    [nkvh][p1-p0][256], then the scales [nkvh][p1-p0][16 B] (Decoder::kv_copy, src/model.cu:1809-1830:
    two strided copies per cache, values first)."""
    cache = np.asarray(cache, np.uint8)
    vals = cache[: nkvh * n_ctx * AD].reshape(nkvh, n_ctx, AD)[:, p0:p1]
    sc = cache[nkvh * n_ctx * AD:].reshape(nkvh, n_ctx, 16)[:, p0:p1]
    return np.concatenate([np.ascontiguousarray(vals).reshape(-1), np.ascontiguousarray(sc).reshape(-1)])


def kv_wire_to_cache(cache, wire, nkvh, n_ctx, p0, p1):
    """Inverse of kv_wire_from_cache, in place (the host-to-device direction of Decoder::kv_copy)."""
    n = p1 - p0
    wire = np.asarray(wire, np.uint8)
    cache[: nkvh * n_ctx * AD].reshape(nkvh, n_ctx, AD)[:, p0:p1] = wire[: nkvh * n * AD].reshape(nkvh, n, AD)
    cache[nkvh * n_ctx * AD:].reshape(nkvh, n_ctx, 16)[:, p0:p1] = wire[nkvh * n * AD:].reshape(nkvh, n, 16)
