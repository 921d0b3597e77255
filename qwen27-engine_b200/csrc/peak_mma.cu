// Peak microbenchmark of the 5th-generation tensor cores for the two kinds the prefill kernels use:
// tcgen05.mma kind::i8 (s8 x s8 -> s32) and kind::f16 (f16 x f16 -> f32), 128 x 256 tiles, operands
// resident in shared memory (no loads in the timed loop), accumulators in tensor memory. The
// reference quotes its prefill kernel against the int8 / f16 tensor peak of its card
// (docs/PERFORMANCE.md:214); this gives the same denominators for this GPU, measured rather than
// taken from a data sheet. No counterpart in the reference.
//
// One CTA per SM, 128 threads. Thread 0 issues `iters` rounds of four MMAs (the four 32-byte k-steps
// of a 128-byte swizzled row: K = 32 for 8-bit operands, K = 16 for 16-bit ones), alternating between
// two accumulators, commits, and waits (bounded) for the commit. Time is taken by the host with
// events around the launch; ops = 2 * 128 * 256 * K per MMA.
#include "common.cuh"
#include "host.h"

namespace q27b {
namespace {

constexpr int PK_A_BYTES = 128 * 128;   // A: 128 rows x 128 bytes, K-major, 128-byte swizzle
constexpr int PK_B_BYTES = 256 * 128;   // B: 256 rows x 128 bytes
constexpr int PK_OFF_BAR = PK_A_BYTES + PK_B_BYTES;
constexpr int PK_SMEM = PK_OFF_BAR + 64 + 1024;
constexpr uint32_t IDESC_I8 = umma_idesc(2, 1, 1, 0, 0, 128, 256);   // s32 += s8 * s8, both K-major
constexpr uint32_t IDESC_F16 = umma_idesc(1, 0, 0, 0, 0, 128, 256);  // f32 += f16 * f16, both K-major

template <bool I8>
__global__ void __launch_bounds__(128, 1) peak_mma_kernel(int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  uint64_t* bar = (uint64_t*)(sgen + PK_OFF_BAR);
  uint32_t* tmem_slot = (uint32_t*)(sgen + PK_OFF_BAR + 32);
  volatile int* abort_flag = (volatile int*)(sgen + PK_OFF_BAR + 36);
  const int tid = threadIdx.x, warp = tid >> 5;
  // operands: small integers (valid in both encodings: as f16 bit patterns they are tiny denormals)
  for (int i = tid; i < (PK_A_BYTES + PK_B_BYTES) / 4; i += 128) ((uint32_t*)sgen)[i] = 0x01010101u * (uint32_t)(i & 3);
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (tid == 0) {
    for (int it = 0; it < iters; it++) {
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const uint64_t da = umma_desc_sw128(sbase + k * 32, 16, 1024);
        const uint64_t db = umma_desc_sw128(sbase + PK_A_BYTES + k * 32, 16, 1024);
        const uint32_t acc = tmem + (it & 1) * 256;
        if (I8) tc_mma_i8(acc, da, db, IDESC_I8, (it > 1 || k > 0) ? 1u : 0u);
        else tc_mma_f16(acc, da, db, IDESC_F16, (it > 1 || k > 0) ? 1u : 0u);
      }
    }
    tc_commit(&bar[0]);
    mbar_wait(&bar[0], 0, abort_flag, status);
  }
  drain_after_abort(abort_flag);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" int q27b_debug_mma_peak(int kind, int iters, void* stream, double* ops_per_launch) {
  if (kind < 0 || kind > 1 || iters < 2 || iters > (1 << 20)) return fail(Q27B_BAD_SHAPE, "debug_mma_peak: kind 0 (i8) or 1 (f16), 2 <= iters <= 2^20");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  static bool attr[64] = {};
  if (!attr[ctx->dev]) {
    Q27B_CK(cudaFuncSetAttribute(peak_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PK_SMEM));
    Q27B_CK(cudaFuncSetAttribute(peak_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PK_SMEM));
    attr[ctx->dev] = true;
  }
  if (kind == 0) peak_mma_kernel<true><<<ctx->n_sm, 128, PK_SMEM, (cudaStream_t)stream>>>(iters, ctx->status);
  else peak_mma_kernel<false><<<ctx->n_sm, 128, PK_SMEM, (cudaStream_t)stream>>>(iters, ctx->status);
  Q27B_CK(cudaGetLastError());
  if (ops_per_launch) *ops_per_launch = 2.0 * 128 * 256 * (kind == 0 ? 32 : 16) * 4.0 * iters * ctx->n_sm;
  return Q27B_OK;
}
