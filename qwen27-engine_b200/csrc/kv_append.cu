// KV append / q8_0 quantise, with the optional q/k RMSNorm + partial RoPE prologue.
//
// Replaces attn_prep_kernel of the reference (src/ops.cu:587-654). One warp owns one row of 256
// values: lane l holds dims 4l..4l+3 and 128+4l..128+4l+3 (two float4 loads, coalesced), so a
// q8_0 block of 32 dims is 8 neighbouring lanes of one half and its amax takes 3 shuffles; the
// quantised row leaves as one 32-bit store per lane and half. This translation unit is built
// WITHOUT fast-math: the q8_0 bytes are specified as IEEE operations
// (d = amax / 127, id = d ? 1 / d : 0, q = roundf(x * id), scale = f16(d); src/ops.cu:636-651)
// and must match the CPU oracle bit for bit.
#include "common.cuh"
#include "host.h"

namespace q27b {
namespace {

struct PrepParams {
  const float* qg;      // [T][nqh][512] (query in the first 256 of each 512) or null
  const float* k;       // [T][nkvh][256]
  const float* v;       // [T][nkvh][256]
  const float* q_norm;  // [256] or null (no norm / RoPE: plain append)
  const float* k_norm;
  float* qn;            // [T][nqh][256]
  void* kcache;
  void* vcache;
  const int* pos0;
  const int* rope3;   // [T][3] or null
  const int* rdelta;  // or null
  int T, nqh, nkvh, n_ctx, q8;
  float eps, theta_scale;
  // Batched form over a page pool (page_table != null): B sequences, T new tokens each at positions
  // seq_len[b] - T + t; qg, k, v, qn carry a leading [B]; rope3 is [B][T][3], rdelta [B].
  const int* page_table;  // [B][max_pages]
  const int* seq_len;     // [B], the new tokens included
  int B, max_pages, n_pages;
  int* status;
};

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// q8_0 of the 4 values of this lane (one of the 8 lanes of a 32-dim block): returns the 4 packed
// int8 and the block scale.
__device__ __forceinline__ uint32_t quant4(const float (&x)[4], float& d_out) {
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
  for (int o = 1; o <= 4; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float d = __fdiv_rn(amax, 127.f);
  const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.0f;
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int q = (int)roundf(__fmul_rn(x[i], id));
    w |= (uint32_t)(q & 0xFF) << (8 * i);
  }
  d_out = d;
  return w;
}

// Writes one row (two float4 halves per lane) to row `row` of a cache (or page pool) of `rows` rows.
__device__ __forceinline__ void store_row(const float (&a)[4], const float (&b)[4], void* cache, size_t row, int lane,
                                          size_t rows, bool q8) {
  if (!q8) {
    __half2* dst = (__half2*)((__half*)cache + row * AD);
    dst[2 * lane] = __floats2half2_rn(a[0], a[1]);
    dst[2 * lane + 1] = __floats2half2_rn(a[2], a[3]);
    dst[64 + 2 * lane] = __floats2half2_rn(b[0], b[1]);
    dst[64 + 2 * lane + 1] = __floats2half2_rn(b[2], b[3]);
    return;
  }
  float da, db;
  const uint32_t wa = quant4(a, da), wb = quant4(b, db);
  uint32_t* vals = (uint32_t*)((uint8_t*)cache + row * AD);
  vals[lane] = wa;
  vals[32 + lane] = wb;
  if ((lane & 7) == 0) {
    __half* sc = (__half*)((uint8_t*)cache + rows * AD) + row * 8;
    sc[lane >> 3] = __float2half_rn(da);
    sc[4 + (lane >> 3)] = __float2half_rn(db);
  }
}

// Grid: ceil(jobs / 8) CTAs of 8 warps; job = (token, row kind). With norm: nqh query rows, then
// nkvh K rows, then nkvh V rows per token; without: K rows then V rows.
__global__ void __launch_bounds__(256) prep_kernel(const PrepParams p) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const bool norm = p.q_norm != nullptr;
  const int per_tok = (norm ? p.nqh : 0) + 2 * p.nkvh;
  const int job = blockIdx.x * 8 + (threadIdx.x >> 5);
  const bool paged = p.page_table != nullptr;
  if (job >= (paged ? p.B : 1) * p.T * per_tok) return;
  const int tok = job / per_tok;  // with pages: sequence * T + token
  int r = job % per_tok;
  const int seq = paged ? tok / p.T : 0;
  const int pos = paged ? p.seq_len[seq] - p.T + tok % p.T : *p.pos0 + tok;
  if (pos < 0 || pos >= p.n_ctx) return;  // never write outside the cache
  const bool isq = norm && r < p.nqh;
  if (norm && !isq) r -= p.nqh;
  const bool isv = !isq && r >= p.nkvh;
  const int head = isq ? r : (isv ? r - p.nkvh : r);
  const float* src = isq ? p.qg + ((size_t)tok * p.nqh + head) * 512
                         : (isv ? p.v : p.k) + ((size_t)tok * p.nkvh + head) * AD;
  const float4 fa = *(const float4*)(src + 4 * lane), fb = *(const float4*)(src + 128 + 4 * lane);
  float a[4] = {fa.x, fa.y, fa.z, fa.w}, b[4] = {fb.x, fb.y, fb.z, fb.w};

  if (norm && !isv) {
    // x * rsqrt(mean(x^2) + eps) * w (src/ops.cu:609-612)
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) t += a[i] * a[i] + b[i] * b[i];
    t = warp_sum(t);
    const float scale = rsqrtf(t / 256 + p.eps);
    const float* w = isq ? p.q_norm : p.k_norm;
    const float4 wa = *(const float4*)(w + 4 * lane), wb = *(const float4*)(w + 128 + 4 * lane);
    const float wav[4] = {wa.x, wa.y, wa.z, wa.w}, wbv[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      a[i] = scale * a[i] * wav[i];
      b[i] = scale * b[i] * wbv[i];
    }
    // NeoX RoPE on pairs (j, j + 32), j < 32: lanes 0..7 hold j = 4l..4l+3, lanes 8..15 the partners
    // (src/ops.cu:614-627). theta = p * theta_scale^j; p = t, h, w of rope3 by j % 3 (IMRoPE).
    float other[4];
#pragma unroll
    for (int i = 0; i < 4; i++) other[i] = __shfl_xor_sync(0xffffffffu, a[i], 8);
    if (lane < 16) {
      const int rp_text = pos - (p.rdelta ? p.rdelta[seq] : 0);
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int j = (4 * lane + i) & 31;
        const int rp = p.rope3 ? p.rope3[tok * 3 + j % 3] : rp_text;
        const float theta = (float)rp * __powf(p.theta_scale, (float)j);
        const float c = __cosf(theta), sn = __sinf(theta);
        const float x0 = lane < 8 ? a[i] : other[i], x1 = lane < 8 ? other[i] : a[i];
        a[i] = lane < 8 ? x0 * c - x1 * sn : x0 * sn + x1 * c;
      }
    }
  }
  if (isq) {
    float* dst = p.qn + ((size_t)tok * p.nqh + head) * AD;
    *(float4*)(dst + 4 * lane) = make_float4(a[0], a[1], a[2], a[3]);
    *(float4*)(dst + 128 + 4 * lane) = make_float4(b[0], b[1], b[2], b[3]);
    return;
  }
  if (!paged) {
    store_row(a, b, isv ? p.vcache : p.kcache, (size_t)head * p.n_ctx + pos, lane, (size_t)p.nkvh * p.n_ctx, p.q8 != 0);
    return;
  }
  const int pg = p.page_table[(size_t)seq * p.max_pages + pos / Q27B_PAGE];
  if (pg < 0 || pg >= p.n_pages) {  // never write outside the pool: flag it and drop the row
    if (lane == 0) atomicOr(p.status, ST_BAD_PAGE);
    return;
  }
  store_row(a, b, isv ? p.vcache : p.kcache, ((size_t)pg * p.nkvh + head) * Q27B_PAGE + pos % Q27B_PAGE, lane,
            (size_t)p.n_pages * p.nkvh * Q27B_PAGE, true);
}

int launch_prep(const PrepParams& p, cudaStream_t s) {
  const int per_tok = (p.q_norm ? p.nqh : 0) + 2 * p.nkvh;
  const int jobs = (p.page_table ? p.B : 1) * p.T * per_tok;
  prep_kernel<<<(jobs + 7) / 8, 256, 0, s>>>(p);
  Q27B_CK(cudaGetLastError());
  return Q27B_OK;
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" {

int q27b_kv_append(const float* k, const float* v, void* kcache, void* vcache, const int* pos0, int T, int nkvh,
                   int n_ctx, int q8, void* stream) {
  if (!k || !v || !kcache || !vcache || !pos0) return fail(Q27B_BAD_SHAPE, "kv_append: null pointer");
  if (T < 1 || nkvh < 1 || n_ctx < 1) return fail(Q27B_BAD_SHAPE, "kv_append: bad shape");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  PrepParams p = {};
  p.k = k; p.v = v; p.kcache = kcache; p.vcache = vcache; p.pos0 = pos0;
  p.T = T; p.nkvh = nkvh; p.n_ctx = n_ctx; p.q8 = q8;
  return launch_prep(p, (cudaStream_t)stream);
}

int q27b_attn_prep(const float* qg, const float* k, const float* v, const float* q_norm, const float* k_norm,
                   float* qn, void* kcache, void* vcache, const int* pos0, int T, float eps, float theta_scale,
                   int nqh, int nkvh, int n_ctx, int q8, void* stream, const int* rope3, const int* rdelta) {
  if (!qg || !k || !v || !q_norm || !k_norm || !qn || !kcache || !vcache || !pos0)
    return fail(Q27B_BAD_SHAPE, "attn_prep: null pointer");
  if (T < 1 || nqh < 1 || nkvh < 1 || n_ctx < 1) return fail(Q27B_BAD_SHAPE, "attn_prep: bad shape");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  PrepParams p = {};
  p.qg = qg; p.k = k; p.v = v; p.q_norm = q_norm; p.k_norm = k_norm; p.qn = qn;
  p.kcache = kcache; p.vcache = vcache; p.pos0 = pos0; p.rope3 = rope3; p.rdelta = rdelta;
  p.T = T; p.nqh = nqh; p.nkvh = nkvh; p.n_ctx = n_ctx; p.q8 = q8; p.eps = eps; p.theta_scale = theta_scale;
  return launch_prep(p, (cudaStream_t)stream);
}

int q27b_attn_prep_paged(const float* qg, const float* k, const float* v, const float* q_norm, const float* k_norm,
                         float* qn, void* kpool, void* vpool, const int* page_table, const int* seq_len, int B, int T,
                         float eps, float theta_scale, int nqh, int nkvh, int n_pages, int max_pages, void* stream,
                         const int* rope3, const int* rdelta) {
  const bool norm = q_norm != nullptr;
  if (!k || !v || !kpool || !vpool || !page_table || !seq_len || (norm && (!qg || !k_norm || !qn)))
    return fail(Q27B_BAD_SHAPE, "attn_prep_paged: null pointer");
  if (B < 1 || T < 1 || nkvh < 1 || n_pages < 1 || max_pages < 1 || max_pages > (1 << 22) || (norm && nqh < 1) ||
      (int64_t)B * T * (nqh + 2 * nkvh) > (int64_t)1 << 30)
    return fail(Q27B_BAD_SHAPE, "attn_prep_paged: bad shape");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  PrepParams p = {};
  p.qg = qg; p.k = k; p.v = v; p.q_norm = q_norm; p.k_norm = norm ? k_norm : nullptr; p.qn = qn;
  p.kcache = kpool; p.vcache = vpool; p.rope3 = rope3; p.rdelta = rdelta;
  p.T = T; p.nqh = nqh; p.nkvh = nkvh; p.n_ctx = max_pages * Q27B_PAGE; p.q8 = 1; p.eps = eps; p.theta_scale = theta_scale;
  p.page_table = page_table; p.seq_len = seq_len; p.B = B; p.max_pages = max_pages; p.n_pages = n_pages;
  p.status = ctx->status;
  return launch_prep(p, (cudaStream_t)stream);
}

}  // extern "C"
