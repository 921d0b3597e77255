// The slow checking kernel of the operator layer: q27::attn_decode_ref (src/ops.h:73-75; kernel and
// host wrapper src/attn.cu:824-867,976-987), which the reference's own check-and-bench tool
// (tools/bench_attn.cu) compares every fast kernel with. Plain softmax over all visible positions
// in f32 with the roundings of the definition: Q * kq_scale -> f16, a cache value = f16(int8 * f16
// scale) (or the stored f16), P = e^(s - max) -> f16 for the P V sum, the row sum from the f32 P.
//
// One CTA per (query head, token). Pass 1: one warp per position, the lanes share the 256 dims
// (coalesced rows, shuffle reduction), scores to a scratch row; pass 2: one thread per output dim
// walks the positions. Meant for checks: T may be any size (the tool passes prefill chunks of 512
// tokens), the scratch (T * nqh * n_ctx floats) is grown on demand and is not part of the workspace
// that q27b_attn_workspace_init fixes.
#include "common.cuh"
#include "host.h"

namespace q27b {
namespace {

__device__ __forceinline__ float cache_value(const void* c, bool q8, size_t row, int i, size_t rows_total) {
  if (!q8) return __half2float(((const __half*)c)[row * AD + i]);
  const int8_t q = ((const int8_t*)c)[row * AD + i];
  const __half d = ((const __half*)((const uint8_t*)c + rows_total * AD))[row * 8 + i / 32];
  return __half2float(__float2half_rn((float)q * __half2float(d)));
}

__global__ void __launch_bounds__(AD) decode_ref_kernel(const float* qn, const float* qg, const void* kc, const void* vc,
                                                         float* o, float* scores, const int* pos0, int nqh, int nkvh, int n_ctx,
                                                         float kq_scale, bool q8) {
  pdl_wait();
  pdl_trigger();
  const int h = blockIdx.x, t = blockIdx.y, d = threadIdx.x, lane = d & 31, warp = d >> 5;
  const int kh = h / GQA;
  const int n = min(n_ctx, *pos0 + t + 1);
  const size_t rows_total = (size_t)nkvh * n_ctx, row0 = (size_t)kh * n_ctx;
  __shared__ float q[AD];
  __shared__ float red[AD / 32];
  q[d] = __half2float(__float2half_rn(qn[((size_t)t * nqh + h) * AD + d] * kq_scale));
  __syncthreads();
  float* sc = scores + ((size_t)t * nqh + h) * n_ctx;
  float mx = -INFINITY;
  for (int p = warp; p < n; p += AD / 32) {
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) a += q[lane * 8 + i] * cache_value(kc, q8, row0 + p, lane * 8 + i, rows_total);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
    if (lane == 0) sc[p] = a;
    mx = fmaxf(mx, a);
  }
  if (lane == 0) red[warp] = mx;
  __syncthreads();  // also makes the scores visible to every thread of the CTA
  mx = red[0];
#pragma unroll
  for (int i = 1; i < AD / 32; i++) mx = fmaxf(mx, red[i]);
  float L = 0.f, A = 0.f;
  for (int p = 0; p < n; p++) {
    const float e = expf(sc[p] - mx);
    L += e;
    A += __half2float(__float2half_rn(e)) * cache_value(vc, q8, row0 + p, d, rows_total);
  }
  const float gate = qg[((size_t)t * nqh + h) * 512 + 256 + d];
  o[((size_t)t * nqh + h) * AD + d] = (A / L) * (1.0f / (1.0f + expf(-gate)));
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" int q27b_attn_decode_ref(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                                    const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8,
                                    void* stream) {
  if (T < 1 || T > 65535 || nkvh < 1 || nqh != nkvh * GQA || n_ctx < 1) return fail(Q27B_BAD_SHAPE, "attn_decode_ref: bad shape");
  if (!qn || !qg || !kcache || !vcache || !o || !pos0) return fail(Q27B_BAD_SHAPE, "attn_decode_ref: null pointer");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  const size_t need = (size_t)T * nqh * n_ctx;
  if (need > ctx->ref_scores_floats) {
    if (ctx->ref_scores) Q27B_CK(cudaFree(ctx->ref_scores));
    ctx->ref_scores = nullptr;
    ctx->ref_scores_floats = 0;
    Q27B_CK(cudaMalloc(&ctx->ref_scores, need * sizeof(float)));
    ctx->ref_scores_floats = need;
  }
  Q27B_CK(launch_pdl(decode_ref_kernel, dim3(nqh, T), dim3(AD), 0, (cudaStream_t)stream, qn, qg, kcache, vcache, o,
                     ctx->ref_scores, pos0, nqh, nkvh, n_ctx, kq_scale, q8 != 0));
  return Q27B_OK;
}
