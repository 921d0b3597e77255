// The step that follows the attention output projection in every layer: x += sum over the GPUs of
// their partial projection rows, then RMSNorm(x) * w -> h (optional) and q8_1 for the next GEMV.
//
// The reference (sum_norm_q8, src/ops.h:101-104; sum_norm_q8_kernel, src/ops.cu:129-260; called
// from src/model.cu:652-692) has two cards on PCIe: the partials cross through mapped host memory in
// a compressed wire format (bf16, or q8 with error feedback), one flag per row, a one-second bound
// on the wait. Here the GPUs share an NVLink switch: every rank stores its f32 rows straight into
// the exchange buffers of all ranks (peer stores of 8-byte words {value, step tag}: no fence, no flag, see
// ll_store), each rank adds the slices in rank order - so every rank gets the same bits - and no wire
// format is needed. As in the decode exchange (combine.cu) the remote rows land in the rank's own memory
// before anything reads them, waits are bounded and end in the status word, and there are no multicast loads.
//
// Numerics of the reference's row kernel (norm_q8_row, src/ops.cu:89-107): t = sum v^2 in f32,
// scale = rsqrtf(t / n + eps) with n a run-time divisor, y = scale * v * w, q8_1 per 32 values as
// q8_store (src/common.cuh:72-81). Thread t holds the values t, t + 1024, ..: the same per-thread
// order of the squares; the tree of the block sum may round differently in the last bit.
#include "combine.h"
#include "common.cuh"
#include "host.h"

namespace q27b {
namespace {

constexpr int SN_THREADS = 1024;
constexpr int SN_MAX_NPT = 16;  // n <= 16384

struct SumNormParams {
  float* x;              // [rows][n] residual stream, updated in place
  const float* partial;  // [rows][n] this rank's partial (no exchange), or null
  const float* w;        // [n]
  float* h;              // [rows][n] or null
  int8_t* xq;            // [rows][n] or null
  float* xd;             // [rows * n / 32]
  int* xbuf;             // exchange buffer of this rank (wait mode), or null
  int* status;
  float eps;
  int rows, n, world;
  // wait mode, fused with the push: this rank's partial rows and the buffers of all ranks as mapped here
  const float* push_src;  // [rows][n] or null
  void* peer[8];
  int rank;
};

__device__ __forceinline__ float block_sum_1024(float t, float* sred) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sred[warp] = t;
  __syncthreads();
  float s = sred[lane];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  return s;
}

// One CTA per row. WAIT: the partials of all ranks are taken from the exchange buffer, word by word, once
// they carry the tag of this step (with push_src: after this rank's own rows have gone out, see below).
template <bool WAIT>
__global__ void __launch_bounds__(SN_THREADS, 1) sum_norm_kernel(const SumNormParams p) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sred[32];
  const int row = blockIdx.x, tid = threadIdx.x, n = p.n;
  const int npt = n / SN_THREADS + (tid < n % SN_THREADS ? 1 : 0);  // n is a multiple of 32, not of 1024
  float v[SN_MAX_NPT];
  float* xr = p.x + (size_t)row * n;
  int epoch = 0;
  if (WAIT) epoch = *(volatile int*)p.xbuf;
  // WAIT: the ranks' rows of this step, words {value, tag} in this rank's own buffer
  const uint64_t* data = WAIT ? (const uint64_t*)((const uint8_t*)p.xbuf + XBUF_HEADER_BYTES) + (size_t)(epoch & 1) * p.world * p.rows * n
                              : nullptr;
  float add[SN_MAX_NPT];
  if (WAIT) {
    bool ok = true;
    float own[SN_MAX_NPT];
    if (p.push_src) {
      // Fused with the push: the grid is (rows, world). CTA (row, dst) with dst != rank stores the row into rank
      // dst's buffer and is done; CTA (row, rank) keeps the row in registers and goes on to wait for the others
      // (every rank's pushes are CTAs of their own, and they come first in the grid: the waiting CTAs have the
      // highest blockIdx.y; the host only takes this form when the whole grid is resident at once, so no
      // wait can hold up a push).
      const int dst = (blockIdx.y + p.rank + 1) % p.world;
#pragma unroll
      for (int k = 0; k < SN_MAX_NPT; k++)
        if (k < npt) {
          const int i = tid + k * SN_THREADS;
          own[k] = p.push_src[(size_t)row * n + i];
          if (dst != p.rank)
            ll_store((uint64_t*)((uint8_t*)p.peer[dst] + XBUF_HEADER_BYTES) +
                         (((size_t)(epoch & 1) * p.world + p.rank) * p.rows + row) * n + i,
                     own[k], epoch + 1);
        }
      if (dst != p.rank) {
        // counted like the waiting CTAs, so that the step only advances once every CTA of the grid has read it
        __syncthreads();
        if (tid == 0 && atomicAdd(p.xbuf + 2, 1) == p.rows * p.world - 1) {
          p.xbuf[2] = 0;
          *(volatile int*)p.xbuf = epoch + 1;
        }
        return;
      }
    }
#pragma unroll
    for (int k = 0; k < SN_MAX_NPT; k++)
      if (k < npt) {
        const int i = tid + k * SN_THREADS;
        float sum = 0.f;
        for (int z = 0; z < p.world; z++) {  // rank order on every rank
          const float t = (p.push_src && z == p.rank) ? own[k] : ll_load(data + ((size_t)z * p.rows + row) * n + i, epoch + 1, ok);
          sum = z == 0 ? t : sum + t;
        }
        add[k] = sum;
      }
    if (__syncthreads_or(!ok)) {  // a rank's rows never arrived: the status word says so, nothing is written
      if (tid == 0 && p.status) atomicOr(p.status, ST_WAIT_EXPIRED);
      return;
    }
  }
  float t = 0.f;
#pragma unroll
  for (int k = 0; k < SN_MAX_NPT; k++) {
    if (k < npt) {
      const int i = tid + k * SN_THREADS;
      const float s = WAIT ? add[k] : p.partial[(size_t)row * n + i];
      v[k] = xr[i] + s;
      xr[i] = v[k];
      t += v[k] * v[k];
    }
  }
  if (WAIT && tid == 0) {
    // the last CTA of the step advances the epoch (nobody reads it again before the next launch)
    if (atomicAdd(p.xbuf + 2, 1) == (p.push_src ? p.rows * p.world : p.rows) - 1) {
      p.xbuf[2] = 0;
      *(volatile int*)p.xbuf = epoch + 1;
    }
  }
  t = block_sum_1024(t, sred);
  const float scale = rsqrtf(t / n + p.eps);
#pragma unroll
  for (int k = 0; k < SN_MAX_NPT; k++) {
    if (k < npt) {  // whole warps: n is a multiple of 32
      const int i = tid + k * SN_THREADS;
      const float y = scale * v[k] * p.w[i];
      const size_t oi = (size_t)row * n + i;
      if (p.h) p.h[oi] = y;
      if (p.xq) {
        float amax = fabsf(y);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float dd = __fdiv_rn(amax, 127.0f);
        p.xq[oi] = amax == 0.0f ? (int8_t)0 : (int8_t)roundf(__fdiv_rn(y, dd));
        if ((tid & 31) == 0) p.xd[oi / 32] = __half2float(__float2half_rn(dd));
      }
    }
  }
}

struct SumPushParams {
  const float* partial;  // [rows][n]
  int* xbuf;             // this rank's own exchange buffer (epoch, counter)
  void* peer[8];         // exchange buffers of all ranks as mapped here (this rank's own among them)
  int rows, n, rank, world;
};

// One CTA per (row, destination rank): the row goes into slot `rank` of that rank's buffer, one tagged 8-byte
// word per value.
__global__ void __launch_bounds__(256) sum_push_kernel(const SumPushParams p) {
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x, k = blockIdx.y, n = p.n;
  const int epoch = *(volatile int*)p.xbuf;
  const float4* src = (const float4*)(p.partial + (size_t)row * n);
  uint64_t* dst = (uint64_t*)((uint8_t*)p.peer[k] + XBUF_HEADER_BYTES) +
                  (((size_t)(epoch & 1) * p.world + p.rank) * p.rows + row) * n;
  for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
    const float4 v = src[i];
    ll_store(dst + 4 * i, v.x, epoch + 1);
    ll_store(dst + 4 * i + 1, v.y, epoch + 1);
    ll_store(dst + 4 * i + 2, v.z, epoch + 1);
    ll_store(dst + 4 * i + 3, v.w, epoch + 1);
  }
}

int check_shape(int rows, int n, const char* who) {
  if (rows < 1 || n < 32 || n % 32 || n > SN_MAX_NPT * SN_THREADS) return fail(Q27B_BAD_SHAPE, who);
  return Q27B_OK;
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" {

uint64_t q27b_sum_xbuf_bytes(int world, int rows, int n) {
  if (world < 1 || rows < 1 || n < 1) return 0;
  return XBUF_HEADER_BYTES + 2ull * (uint64_t)world * (uint64_t)rows * (uint64_t)n * sizeof(uint64_t);  // {value, tag} words
}

int q27b_xbuf_alloc_bytes(uint64_t bytes, void** out) {
  if (!out || bytes < XBUF_HEADER_BYTES) return fail(Q27B_BAD_SHAPE, "xbuf_alloc_bytes: bad size");
  void* p = nullptr;
  Q27B_CK(cudaMalloc(&p, bytes));  // an allocation of its own: an IPC handle names whole allocations
  Q27B_CK(cudaMemset(p, 0, bytes));
  Q27B_CK(cudaDeviceSynchronize());
  *out = p;
  return Q27B_OK;
}

int q27b_sum_norm_q8(float* x, const float* partial, int n, int rows, const float* w, float eps, float* h, int8_t* xq,
                     float* xd, void* stream) {
  if (!x || !partial || !w || (xq && !xd)) return fail(Q27B_BAD_SHAPE, "sum_norm_q8: null pointer");
  if (int rc = check_shape(rows, n, "sum_norm_q8: rows >= 1, n a multiple of 32 up to 16384")) return rc;
  SumNormParams p = {};
  p.x = x; p.partial = partial; p.w = w; p.h = h; p.xq = xq; p.xd = xd; p.eps = eps; p.rows = rows; p.n = n; p.world = 1;
  Q27B_CK(launch_pdl(sum_norm_kernel<false>, dim3(rows), dim3(SN_THREADS), 0, (cudaStream_t)stream, p));
  return Q27B_OK;
}

int q27b_sum_push(const float* partial, int n, int rows, int rank, int world, void* const* xbufs, void* stream) {
  if (!partial || !xbufs) return fail(Q27B_BAD_SHAPE, "sum_push: null pointer");
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(Q27B_BAD_SHAPE, "sum_push: bad rank/world");
  if (int rc = check_shape(rows, n, "sum_push: rows >= 1, n a multiple of 32 up to 16384")) return rc;
  SumPushParams p = {};
  p.partial = partial; p.rows = rows; p.n = n; p.rank = rank; p.world = world;
  for (int k = 0; k < world; k++)
    if (!xbufs[k]) return fail(Q27B_BAD_SHAPE, "sum_push: null exchange buffer");
  // Every buffer must be device memory that kernels of this GPU may store into (its own, or a peer's
  // with peer access, enabled here once per pointer); anything else is refused before the launch.
  for (int k = 0; k < world; k++) {
    if (int rc = check_peer_buffer(xbufs[k], "sum_push")) return rc;
    p.peer[k] = xbufs[k];
  }
  p.xbuf = (int*)xbufs[rank];
  Q27B_CK(launch_pdl(sum_push_kernel, dim3(rows, world), dim3(256), 0, (cudaStream_t)stream, p));
  return Q27B_OK;
}

int q27b_sum_norm_q8_wait(float* x, void* xbuf, int world, int n, int rows, const float* w, float eps, float* h, int8_t* xq,
                          float* xd, void* stream) {
  if (!x || !xbuf || !w || (xq && !xd)) return fail(Q27B_BAD_SHAPE, "sum_norm_q8_wait: null pointer");
  if (world < 1 || world > 8) return fail(Q27B_BAD_SHAPE, "sum_norm_q8_wait: 1..8 ranks");
  if (int rc = check_shape(rows, n, "sum_norm_q8_wait: rows >= 1, n a multiple of 32 up to 16384")) return rc;
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  SumNormParams p = {};
  p.x = x; p.w = w; p.h = h; p.xq = xq; p.xd = xd; p.eps = eps; p.rows = rows; p.n = n; p.world = world;
  p.xbuf = (int*)xbuf; p.status = ctx->status;
  Q27B_CK(launch_pdl(sum_norm_kernel<true>, dim3(rows), dim3(SN_THREADS), 0, (cudaStream_t)stream, p));
  return Q27B_OK;
}

int q27b_sum_exchange_norm_q8(float* x, const float* partial, int n, int rows, int rank, int world, void* const* xbufs,
                              const float* w, float eps, float* h, int8_t* xq, float* xd, void* stream) {
  if (!x || !partial || !xbufs || !w || (xq && !xd)) return fail(Q27B_BAD_SHAPE, "sum_exchange_norm_q8: null pointer");
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(Q27B_BAD_SHAPE, "sum_exchange_norm_q8: bad rank/world");
  if (int rc = check_shape(rows, n, "sum_exchange_norm_q8: rows >= 1, n a multiple of 32 up to 16384")) return rc;
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  SumNormParams p = {};
  p.x = x; p.w = w; p.h = h; p.xq = xq; p.xd = xd; p.eps = eps; p.rows = rows; p.n = n; p.world = world;
  p.push_src = partial; p.rank = rank; p.status = ctx->status;
  for (int k = 0; k < world; k++) {
    if (!xbufs[k]) return fail(Q27B_BAD_SHAPE, "sum_exchange_norm_q8: null exchange buffer");
    if (int rc = check_peer_buffer(xbufs[k], "sum_exchange_norm_q8")) return rc;
    p.peer[k] = xbufs[k];
  }
  p.xbuf = (int*)xbufs[rank];
  if ((int64_t)rows * world > ctx->n_sm) {  // more CTAs than are resident at once: push, then wait, as two launches
    if (int rc = q27b_sum_push(partial, n, rows, rank, world, xbufs, stream)) return rc;
    return q27b_sum_norm_q8_wait(x, xbufs[rank], world, n, rows, w, eps, h, xq, xd, stream);
  }
  Q27B_CK(launch_pdl(sum_norm_kernel<true>, dim3(rows, world), dim3(SN_THREADS), 0, (cudaStream_t)stream, p));
  return Q27B_OK;
}

}  // extern "C"
