// CPU restatement of the attention hot path of avallavall/qwen27-engine.
//
// TEST INFRASTRUCTURE ONLY. This file is the checker: tests, the smoke check and the
// cpu_baseline leg of the benchmark call it. The shipped library never links or loads it.
//
// Parity status: the reference holds no golden vectors for this path (its only check,
// tools/bench_attn.cu, prints a max error against its own slow GPU kernel). The functions
// below are therefore pinned against outputs of the reference's own kernels, compiled from the
// reference sources for sm_100a and run on a B200 on seeded inputs; those outputs are the
// fixtures under tests/golden/ (made by tests/golden/make_golden.py).
//
// Every function cites the reference lines it restates. Plain C++17 + OpenMP, IEEE arithmetic
// (build with -ffp-contract=off so the quantisers are reproducible bit for bit).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr int AD = 256;   // head dim (src/attn.cu:22)
constexpr int GQA = 6;    // query heads per KV head (src/attn.cu:23)
constexpr int PROW = AD + 2;  // floats of one partial row: m, l, O[256] (src/attn.cu:26)
constexpr float M_INIT = -1e30f;  // src/attn.cu:28

inline float h2f(uint16_t h) {
  _Float16 x;
  std::memcpy(&x, &h, 2);
  return (float)x;
}
inline uint16_t f2h(float f) {  // round to nearest even, as __float2half
  _Float16 x = (_Float16)f;
  uint16_t h;
  std::memcpy(&h, &x, 2);
  return h;
}
inline float rh(float f) { return (float)(_Float16)f; }  // round through f16

// One element of a cache row as the kernels see it: f16 value, or f16(int8 * f16 scale)
// (cache_val, src/attn.cu:827-832). Row layout: src/ops.h:50-53.
inline void load_row(const void* c, bool q8, int nkvh, int n_ctx, int kh, int p, float* out) {
  const size_t row = (size_t)kh * n_ctx + p;
  if (!q8) {
    const uint16_t* h = (const uint16_t*)c + row * AD;
    for (int i = 0; i < AD; i++) out[i] = h2f(h[i]);
    return;
  }
  const int8_t* q = (const int8_t*)c + row * AD;
  const uint16_t* d = (const uint16_t*)((const uint8_t*)c + (size_t)nkvh * n_ctx * AD) + row * 8;
  for (int b = 0; b < 8; b++) {
    const float db = h2f(d[b]);
    for (int i = 0; i < 32; i++) out[b * 32 + i] = rh((float)q[b * 32 + i] * db);
  }
}

inline float sigmoidf(float g) { return 1.0f / (1.0f + std::exp(-g)); }

}  // namespace

extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Bytes of the K (or V) cache of one layer (kv_cache_bytes, src/attn.cu:890-892).
uint64_t orc_kv_cache_bytes(int nkvh, int n_ctx, int q8) {
  return q8 ? (uint64_t)nkvh * n_ctx * (AD + 16) : (uint64_t)nkvh * n_ctx * AD * 2;
}

// q8_0 of `rows` rows of 256 floats: per 32 values d = amax / 127, id = d ? 1/d : 0,
// q = (int8) roundf(x * id) (half away from zero), scale stored as f16(d)
// (attn_prep_kernel, src/ops.cu:636-651).
void orc_quant_q8_0(const float* x, int64_t rows, int8_t* q, uint16_t* d) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++)
    for (int b = 0; b < 8; b++) {
      const float* s = x + r * AD + b * 32;
      float amax = 0.f;
      for (int i = 0; i < 32; i++) amax = std::fmax(amax, std::fabs(s[i]));
      const float dd = amax / 127.f;
      const float id = dd ? 1.0f / dd : 0.0f;
      for (int i = 0; i < 32; i++) q[r * AD + b * 32 + i] = (int8_t)std::round(s[i] * id);
      d[r * 8 + b] = f2h(dd);
    }
}

// K/V rows of T tokens ([T][nkvh][256] f32) written at cache rows pos0 + t, q8_0 or f16
// (tail of attn_prep_kernel, src/ops.cu:628-652; K here is the row after norm and RoPE).
void orc_kv_append(const float* k, const float* v, void* kcache, void* vcache, int pos0, int T, int nkvh,
                   int n_ctx, int q8) {
  for (int w = 0; w < 2; w++) {
    const float* src = w ? v : k;
    uint8_t* cache = (uint8_t*)(w ? vcache : kcache);
    for (int t = 0; t < T; t++)
      for (int kh = 0; kh < nkvh; kh++) {
        const float* x = src + ((size_t)t * nkvh + kh) * AD;
        const size_t row = (size_t)kh * n_ctx + pos0 + t;
        if (!q8) {
          uint16_t* dst = (uint16_t*)cache + row * AD;
          for (int i = 0; i < AD; i++) dst[i] = f2h(x[i]);
        } else {
          orc_quant_q8_0(x, 1, (int8_t*)cache + row * AD,
                         (uint16_t*)(cache + (size_t)nkvh * n_ctx * AD) + row * 8);
        }
      }
  }
}

// q8_1 of n values (n % 32 == 0): per 32, d = amax / 127, q = amax == 0 ? 0 : roundf(y / d),
// xd = float(f16(d)) (q8_store, src/common.cuh:72-81).
void orc_q8_1(const float* y, int64_t n, int8_t* xq, float* xd) {
  for (int64_t b = 0; b < n / 32; b++) {
    float amax = 0.f;
    for (int i = 0; i < 32; i++) amax = std::fmax(amax, std::fabs(y[b * 32 + i]));
    const float d = amax / 127.0f;
    for (int i = 0; i < 32; i++) xq[b * 32 + i] = amax == 0.0f ? 0 : (int8_t)std::round(y[b * 32 + i] / d);
    xd[b] = rh(d);
  }
}

// Attention of T query tokens at positions pos0 + t with the decode numerics of the reference's
// slow kernel (attn_ref_kernel, src/attn.cu:833-867): q = f16(qn * scale); s = sum q_i K_i in
// f32; e = exp(s - max); L = sum e; A = sum f16(e) V; o = (A / L) * sigmoid(gate). Token t sees
// positions 0 .. pos0 + t (src/attn.cu:840). qn [T][nqh][256], qg [T][nqh][512] (gate in the
// second half, src/attn.cu:865), o [T][nqh][256].
// With part != null the result is left unnormalised instead: part [T][nqh][258] = (max, L, A),
// restricted to positions [p_lo, p_hi) (the split the kernels merge, src/attn.cu:286-289).
static void attn_rows(const float* qn, const float* qg, const void* kc, const void* vc, float* o, float* part,
                      int pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, int p_lo, int p_hi) {
  const int n_all = std::min(pos0 + T, p_hi);
  const int np = std::max(0, n_all - p_lo);
  const int R = GQA * T;
  std::vector<float> sc((size_t)nkvh * R * std::max(np, 1));
  for (int kh = 0; kh < nkvh; kh++) {
    std::vector<float> q((size_t)R * AD);
    for (int r = 0; r < R; r++) {
      const int t = r / GQA, h = kh * GQA + r % GQA;
      for (int i = 0; i < AD; i++) q[(size_t)r * AD + i] = rh(qn[((size_t)t * nqh + h) * AD + i] * kq_scale);
    }
    float* s = sc.data() + (size_t)kh * R * std::max(np, 1);
#pragma omp parallel
    {
      float row[AD];
#pragma omp for schedule(static)
      for (int pi = 0; pi < np; pi++) {
        load_row(kc, q8, nkvh, n_ctx, kh, p_lo + pi, row);
        for (int r = 0; r < R; r++) {
          const float* qq = q.data() + (size_t)r * AD;
          float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int i = 0; i < AD; i += 8)
            for (int j = 0; j < 8; j++) a[j] += qq[i + j] * row[i + j];
          s[(size_t)r * np + pi] = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
        }
      }
    }
    // visible positions of row r: p < pos0 + t + 1
    std::vector<float> mx(R, -INFINITY);
    for (int r = 0; r < R; r++) {
      const int vis = std::min(np, pos0 + r / GQA + 1 - p_lo);
      for (int pi = 0; pi < vis; pi++) mx[r] = std::fmax(mx[r], s[(size_t)r * np + pi]);
    }
    int nthr = 1;
#ifdef _OPENMP
    nthr = omp_get_max_threads();
#endif
    std::vector<double> A((size_t)nthr * R * AD, 0.0), L((size_t)nthr * R, 0.0);
#pragma omp parallel
    {
      int tid = 0;
#ifdef _OPENMP
      tid = omp_get_thread_num();
#endif
      double* a = A.data() + (size_t)tid * R * AD;
      double* l = L.data() + (size_t)tid * R;
      float row[AD];
#pragma omp for schedule(static)
      for (int pi = 0; pi < np; pi++) {
        load_row(vc, q8, nkvh, n_ctx, kh, p_lo + pi, row);
        for (int r = 0; r < R; r++) {
          if (p_lo + pi >= pos0 + r / GQA + 1) continue;
          const float e = std::exp(s[(size_t)r * np + pi] - mx[r]);
          l[r] += e;
          const float eh = rh(e);
          double* ar = a + (size_t)r * AD;
          for (int i = 0; i < AD; i++) ar[i] += (double)(eh * row[i]);
        }
      }
    }
    for (int r = 0; r < R; r++) {
      const int t = r / GQA, h = kh * GQA + r % GQA;
      double l = 0;
      for (int k = 0; k < nthr; k++) l += L[(size_t)k * R + r];
      for (int i = 0; i < AD; i++) {
        double a = 0;
        for (int k = 0; k < nthr; k++) a += A[((size_t)k * R + r) * AD + i];
        if (part) {
          part[((size_t)t * nqh + h) * PROW + 2 + i] = (float)a;
        } else {
          const float gate = qg[((size_t)t * nqh + h) * 512 + 256 + i];
          o[((size_t)t * nqh + h) * AD + i] = ((float)a / (float)l) * sigmoidf(gate);
        }
      }
      if (part) {
        const bool empty = !(mx[r] > -INFINITY);
        part[((size_t)t * nqh + h) * PROW] = empty ? M_INIT : mx[r];
        part[((size_t)t * nqh + h) * PROW + 1] = (float)l;
      }
    }
  }
}

void orc_attn_ref(const float* qn, const float* qg, const void* kc, const void* vc, float* o, int pos0, int T,
                  float kq_scale, int nqh, int nkvh, int n_ctx, int q8) {
  attn_rows(qn, qg, kc, vc, o, nullptr, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8, 0, pos0 + T);
}

void orc_attn_partial(const float* qn, const void* kc, const void* vc, float* part, int pos0, int T, float kq_scale,
                      int nqh, int nkvh, int n_ctx, int q8, int p_lo, int p_hi) {
  attn_rows(qn, nullptr, kc, vc, nullptr, part, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8, p_lo, p_hi);
}

// Log-sum-exp merge of nparts partials of `rows` rows, each (m, l, O[256]) with a stride of
// part_stride floats between partials: M = max m; L = sum l e^(m-M); A = sum O e^(m-M);
// y = (A / L) * sigmoid(gate) (attn_combine_kernel, src/attn.cu:302-312; attn_pf_combine_kernel,
// src/attn.cu:811-821). part row r of partial c at part + c * part_stride + r * 258;
// gate of row r at qg + r * 512 + 256 (null: no gate); o [rows][256].
void orc_lse_merge(const float* part, int nparts, int64_t part_stride, int64_t rows, const float* qg, float* o) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++) {
    const float* p = part + r * PROW;
    float M = M_INIT;
    for (int c = 0; c < nparts; c++) M = std::fmax(M, p[c * part_stride]);
    std::vector<float> f(nparts);
    float L = 0.f;
    for (int c = 0; c < nparts; c++) {
      f[c] = std::exp(p[c * part_stride] - M);
      L += p[c * part_stride + 1] * f[c];
    }
    for (int i = 0; i < AD; i++) {
      float A = 0.f;
      for (int c = 0; c < nparts; c++) A += p[c * part_stride + 2 + i] * f[c];
      const float g = qg ? sigmoidf(qg[r * 512 + 256 + i]) : 1.0f;
      o[r * AD + i] = (A / L) * g;
    }
  }
}

// int8 quantiser of the prefill query rows: v = q * kq_scale; per 32 dims amax; d = amax / 127
// (kept in f32), id = amax > 0 ? 127 / amax : 0; q8 = rint(v * id) (half to even)
// (attn_prefill_i8_kernel, src/attn.cu:587-606). x [rows][256] -> q [rows][256], d [rows][8].
void orc_quant_q_i8(const float* x, int64_t rows, float kq_scale, int8_t* q, float* d) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++)
    for (int b = 0; b < 8; b++) {
      float v[32];
      float amax = 0.f;
      for (int i = 0; i < 32; i++) {
        v[i] = x[r * AD + b * 32 + i] * kq_scale;
        amax = std::fmax(amax, std::fabs(v[i]));
      }
      const float id = amax > 0.f ? 127.f / amax : 0.f;
      for (int i = 0; i < 32; i++) q[r * AD + b * 32 + i] = (int8_t)std::nearbyint(v[i] * id);
      d[r * 8 + b] = amax / 127.f;
    }
}

// Per-32-block integer dot products I_b[r][p] = sum_{i in block b} q[r][i] * k[p][i]
// (the int32 accumulators of mma_k32_i8, src/attn.cu:690-691). out [rows][npos][8].
void orc_qk_i32(const int8_t* q, const int8_t* k, int rows, int npos, int32_t* out) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; r++)
    for (int p = 0; p < npos; p++)
      for (int b = 0; b < 8; b++) {
        int32_t a = 0;
        for (int i = 0; i < 32; i++) a += (int32_t)q[(size_t)r * AD + b * 32 + i] * (int32_t)k[(size_t)p * AD + b * 32 + i];
        out[((size_t)r * npos + p) * 8 + b] = a;
      }
}

// Prefill attention with the int8 Q K^T numerics (attn_prefill_i8_kernel, src/attn.cu:557-801):
// Q rows quantised as orc_quant_q_i8; K = the int8 bytes of the q8_0 cache; s = sum over blocks
// in order b = 0..7 of (dq[b] * dk[p][b]) * float(I_b) in f32 (src/attn.cu:682-699); token t sees
// p < pos0 + t + 1 (src/attn.cu:646); P = exp(s - max) rounded to f16 for P V, row sum from the
// f32 P; V = f16(int8 * scale); o = (A / L) * sigmoid(gate) (src/attn.cu:781-800). The exact
// global max is used and O accumulates in f64: the reference's running max with offset and its
// f16 accumulation of O are sources of error of that kernel, not part of the definition.
// Only rows of tokens t in [t_lo, t_hi) are computed (others left untouched).
void orc_attn_prefill_i8(const float* qn, const float* qg, const void* kc, const void* vc, float* o, int pos0, int M,
                         float kq_scale, int nqh, int nkvh, int n_ctx, int t_lo, int t_hi) {
  t_lo = std::max(0, t_lo);
  t_hi = std::min(M, t_hi);
  const int n_max = pos0 + t_hi;
  const int8_t* kq = (const int8_t*)kc;
  const uint16_t* kd = (const uint16_t*)((const uint8_t*)kc + (size_t)nkvh * n_ctx * AD);
  for (int kh = 0; kh < nkvh; kh++) {
    // V rows dequantised once per KV head
    std::vector<float> vf((size_t)n_max * AD);
#pragma omp parallel for schedule(static)
    for (int p = 0; p < n_max; p++) load_row(vc, true, nkvh, n_ctx, kh, p, vf.data() + (size_t)p * AD);
    std::vector<float> dkf((size_t)n_max * 8);
    for (int p = 0; p < n_max; p++)
      for (int b = 0; b < 8; b++) dkf[(size_t)p * 8 + b] = h2f(kd[((size_t)kh * n_ctx + p) * 8 + b]);
    const int nrows = (t_hi - t_lo) * GQA;
#pragma omp parallel
    {
      std::vector<float> s(n_max);
      std::vector<double> acc(AD);
#pragma omp for schedule(dynamic, 1)
      for (int ri = 0; ri < nrows; ri++) {
        const int t = t_lo + ri / GQA, h = kh * GQA + ri % GQA;
        int8_t q8[AD];
        float dq[8];
        orc_quant_q_i8(qn + ((size_t)t * nqh + h) * AD, 1, kq_scale, q8, dq);
        const int n = pos0 + t + 1;
        float mx = -INFINITY;
        for (int p = 0; p < n; p++) {
          const int8_t* kr = kq + ((size_t)kh * n_ctx + p) * AD;
          float sv = 0.f;
          for (int b = 0; b < 8; b++) {
            int32_t ci = 0;
            for (int i = 0; i < 32; i++) ci += (int32_t)q8[b * 32 + i] * (int32_t)kr[b * 32 + i];
            sv += (dq[b] * dkf[(size_t)p * 8 + b]) * (float)ci;
          }
          s[p] = sv;
          mx = std::fmax(mx, sv);
        }
        double L = 0;
        std::fill(acc.begin(), acc.end(), 0.0);
        for (int p = 0; p < n; p++) {
          const float e = std::exp(s[p] - mx);
          L += e;
          const float eh = rh(e);
          const float* vr = vf.data() + (size_t)p * AD;
          for (int i = 0; i < AD; i++) acc[i] += (double)(eh * vr[i]);
        }
        for (int i = 0; i < AD; i++) {
          const float gate = qg[((size_t)t * nqh + h) * 512 + 256 + i];
          o[((size_t)t * nqh + h) * AD + i] = ((float)acc[i] / (float)L) * sigmoidf(gate);
        }
      }
    }
  }
}

}  // extern "C"
