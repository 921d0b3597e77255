// Host-side state and the entry points that launch nothing.
#include "host.h"

#include "common.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace q27b {

namespace {
thread_local std::string g_err;
DeviceCtx g_ctx[64];

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
}  // namespace

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("Q27_PDL");
    return e && e[0] == '1';
  }();
  return on;
}

int fail(int code, const std::string& msg) {
  g_err = msg;
  return code;
}
void clear_error() { g_err.clear(); }
const char* g_err_text() { return g_err.c_str(); }

int device_ctx(DeviceCtx** out) {
  int dev;
  Q27B_CK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(Q27B_UNSUPPORTED, "device index out of range");
  DeviceCtx& c = g_ctx[dev];
  if (c.dev < 0) {
    int major = 0, minor = 0;
    Q27B_CK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    Q27B_CK(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
    if (major != 10) return fail(Q27B_UNSUPPORTED, "q27b_attn is built for sm_100a only; device is sm_" +
                                                       std::to_string(major) + std::to_string(minor));
    Q27B_CK(cudaDeviceGetAttribute(&c.n_sm, cudaDevAttrMultiProcessorCount, dev));
    Q27B_CK(cudaMalloc(&c.status, 256));
    Q27B_CK(cudaMemset(c.status, 0, 256));
    c.dev = dev;
  }
  *out = &c;
  return Q27B_OK;
}

int ensure_part(DeviceCtx* ctx, size_t floats) {
  if (floats <= ctx->part_floats) return Q27B_OK;
  if (ctx->part) Q27B_CK(cudaFree(ctx->part));
  ctx->part = nullptr;
  ctx->part_floats = 0;
  Q27B_CK(cudaMalloc(&ctx->part, floats * sizeof(float)));
  ctx->part_floats = floats;
  return Q27B_OK;
}

int ensure_work(DeviceCtx* ctx, size_t ints) {
  if (ints <= ctx->work_ints) return Q27B_OK;
  if (ctx->work) Q27B_CK(cudaFree(ctx->work));
  ctx->work = nullptr;
  ctx->work_ints = 0;
  Q27B_CK(cudaMalloc(&ctx->work, ints * sizeof(int)));
  ctx->work_ints = ints;
  return Q27B_OK;
}

int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint32_t row_bytes, uint64_t pitch_bytes,
                 uint32_t box_bytes, uint32_t box_rows, bool swizzle128) {
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    Q27B_CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess) return fail(Q27B_CUDA_ERROR, "cuTensorMapEncodeTiled not available");
    g_encode = (EncodeFn)fn;
  }
  if (((uintptr_t)base & 15) != 0) return fail(Q27B_BAD_SHAPE, "cache pointer must be 16-byte aligned");
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_bytes, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(Q27B_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return Q27B_OK;
}

}  // namespace q27b

using namespace q27b;

extern "C" {

const char* q27b_last_error(void) { return g_err_text(); }

int q27b_device_status(int* status_out) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  int st = 0;
  Q27B_CK(cudaDeviceSynchronize());
  Q27B_CK(cudaMemcpy(&st, ctx->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (st) Q27B_CK(cudaMemset(ctx->status, 0, 256));  // the word, and the tile counters an aborted kernel may have left behind
  if (status_out) *status_out = st;
  return st ? fail(Q27B_DEVICE_STATUS, "device status word = " + std::to_string(st)) : Q27B_OK;
}

// One CTA, one warp: waits on an mbarrier that nobody arrives at, with the same bounded wait the
// attention kernels use. The wait gives up after its limit, records ST_WAIT_EXPIRED and the kernel
// returns normally: what a lost signal looks like to the host, without a hang and without a trap.
__global__ void expire_wait_kernel(int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    q27b::mbar_init(&bar, 1);
    abort_flag = 0;
    q27b::mbar_fence_init();
  }
  __syncthreads();
  q27b::mbar_wait(&bar, 0, &abort_flag, status);
  q27b::drain_after_abort(&abort_flag);
}

int q27b_debug_expire_wait(void* stream) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  expire_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ctx->status);
  Q27B_CK(cudaGetLastError());
  return Q27B_OK;
}

// ---- exchange buffers of the peer-memory merge, and their mapping between processes
int q27b_xbuf_alloc(int nz, int64_t rows, void** out) {
  if (!out || nz < 1 || nz > 8 || rows < 1) return fail(Q27B_BAD_SHAPE, "xbuf_alloc: bad shape");
  const size_t bytes = 256 + 2ull * (size_t)nz * (size_t)rows * (Q27B_HEAD_DIM + 2) * sizeof(float);
  void* p = nullptr;
  Q27B_CK(cudaMalloc(&p, bytes));  // an allocation of its own: an IPC handle names whole allocations
  Q27B_CK(cudaMemset(p, 0, bytes));
  Q27B_CK(cudaDeviceSynchronize());
  *out = p;
  return Q27B_OK;
}

int q27b_xbuf_free(void* p) {
  if (p) Q27B_CK(cudaFree(p));
  return Q27B_OK;
}

int q27b_ipc_export(const void* ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr || !handle) return fail(Q27B_BAD_SHAPE, "ipc_export: null pointer");
  cudaIpcMemHandle_t h;
  Q27B_CK(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
  memcpy(handle, &h, 64);
  return Q27B_OK;
}

// Maps a peer's buffer into the address space of the CURRENT device (the one whose kernels will store
// into it), with peer access enabled as part of the mapping. A handle opened while another device is
// current is not reachable from this one, whatever is enabled afterwards.
int q27b_ipc_open(const unsigned char handle[64], void** out) {
  if (!handle || !out) return fail(Q27B_BAD_SHAPE, "ipc_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  Q27B_CK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return Q27B_OK;
}

int q27b_ipc_close(void* p) {
  if (p) Q27B_CK(cudaIpcCloseMemHandle(p));
  return Q27B_OK;
}

uint64_t q27b_kv_cache_bytes(int nkvh, int n_ctx, int q8) {
  return q8 ? (uint64_t)nkvh * n_ctx * (Q27B_HEAD_DIM + 16) : (uint64_t)nkvh * n_ctx * Q27B_HEAD_DIM * 2;
}

uint64_t q27b_kv_pool_bytes(int nkvh, int n_pages) {
  return (uint64_t)n_pages * nkvh * Q27B_PAGE * (Q27B_HEAD_DIM + 16);
}

int q27b_attn_chunks(int nkvh) {
  DeviceCtx* ctx;
  if (nkvh < 1 || device_ctx(&ctx)) return 0;
  return std::max(1, ctx->n_sm / nkvh);
}

}  // extern "C"
