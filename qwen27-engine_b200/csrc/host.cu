// Host-side state and the entry points that launch nothing.
#include "host.h"

#include "common.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

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

namespace {
// Default cap of the prefill partial buffer: 128 MiB. The metric's chunk (2048 tokens, 24 heads) on a
// 148,000-token prefix cuts 4 query tiles into 5 pieces = 63 MB; a chunk whose q8_1 output needs every
// tile on the split path, 2 x 2048 x 24 rows = 101 MB. (The reference fixes 24 MB on a 16 GB card.)
constexpr size_t PF_CAP_DEFAULT_FLOATS = (128ull << 20) / sizeof(float);

int alloc_ws(DeviceCtx* ctx, WsBuf* b, size_t floats, const char* what) {
  if (ctx->frozen)
    return fail(Q27B_UNSUPPORTED, std::string(what) + ": the workspace was fixed by q27b_attn_workspace_init and holds " +
                                      std::to_string(b->floats * sizeof(float)) + " bytes, this call needs " +
                                      std::to_string(floats * sizeof(float)));
  if (b->p) Q27B_CK(cudaFree(b->p));
  b->p = nullptr;
  b->floats = 0;
  Q27B_CK(cudaMalloc(&b->p, floats * sizeof(float)));
  b->floats = floats;
  return Q27B_OK;
}
}  // namespace

int decode_ws(DeviceCtx* ctx, float** out) {
  const size_t need = (size_t)ctx->n_sm * MAXR * PROW;
  if (ctx->dec.floats < need)
    if (int rc = alloc_ws(ctx, &ctx->dec, need, "attn_decode")) return rc;
  *out = ctx->dec.p;
  return Q27B_OK;
}

int prefill_ws(DeviceCtx* ctx, float** out, size_t* max_floats) {
  if (!ctx->pf.p) {
    const size_t cap = ctx->pf_cap_floats ? ctx->pf_cap_floats : PF_CAP_DEFAULT_FLOATS;
    if (int rc = alloc_ws(ctx, &ctx->pf, cap, "attn_prefill")) return rc;
  }
  *out = ctx->pf.p;
  *max_floats = ctx->pf.floats;
  return Q27B_OK;
}

int paged_ws(DeviceCtx* ctx, size_t floats, float** out) {
  if (ctx->paged.floats < floats)
    if (int rc = alloc_ws(ctx, &ctx->paged, floats, "attn_decode_paged")) return rc;
  *out = ctx->paged.p;
  return Q27B_OK;
}

int fit_prefill_split(DeviceCtx* ctx, int* ts, int* ns, int M, int nqh, bool must_merge, float** part) {
  *part = nullptr;
  if (*ns <= 1) return Q27B_OK;
  size_t cap = 0;
  if (int rc = prefill_ws(ctx, part, &cap)) return rc;
  const size_t per_piece = (size_t)std::min(M, *ts * 128) * nqh * PROW;
  const int fit = (int)std::min<size_t>(64, cap / per_piece);
  if (*ns > fit) *ns = fit;
  if (*ns < 2) {
    if (must_merge)
      return fail(Q27B_UNSUPPORTED, "attn_prefill: the prefill workspace (" + std::to_string(cap * sizeof(float)) +
                                        " bytes) is too small for two partials of this call (" +
                                        std::to_string(2 * per_piece * sizeof(float)) + " bytes)");
    *ns = 1;
    *ts = 0;
    *part = nullptr;
  }
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

namespace {
struct TmapKey {
  const void* base;
  uint64_t rows, pitch;
  uint32_t row_bytes, box_bytes, box_rows;
  int swz, dev;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && pitch == o.pitch && row_bytes == o.row_bytes && box_bytes == o.box_bytes &&
           box_rows == o.box_rows && swz == o.swz && dev == o.dev;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = (uint64_t)(uintptr_t)k.base * 0x9E3779B97F4A7C15ull;
    h ^= (k.rows + 0x7F4A7C15ull) * 0xBF58476D1CE4E5B9ull;
    h ^= ((uint64_t)k.row_bytes << 40) ^ ((uint64_t)k.box_bytes << 24) ^ ((uint64_t)k.box_rows << 8) ^ (uint64_t)(k.swz * 2 + k.dev * 4);
    return (size_t)(h ^ (h >> 29));
  }
};
std::mutex g_tmap_mu;
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;
constexpr size_t TMAP_CACHE_MAX = 4096;  // far above what an engine holds (the reference: 17 layers x K, V x 2 cards)

std::mutex g_peer_mu;
std::vector<std::pair<int, const void*>> g_peer_ok;  // (storing device, buffer) pairs already checked
}  // namespace

int cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint32_t row_bytes, uint64_t pitch_bytes,
                   uint32_t box_bytes, uint32_t box_rows, bool swizzle128) {
  int dev = 0;
  Q27B_CK(cudaGetDevice(&dev));
  const TmapKey key = {base, rows, pitch_bytes, row_bytes, box_bytes, box_rows, swizzle128 ? 1 : 0, dev};
  {
    std::lock_guard<std::mutex> lock(g_tmap_mu);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *out = it->second;
      return Q27B_OK;
    }
  }
  if (int rc = make_tmap_2d(out, base, rows, row_bytes, pitch_bytes, box_bytes, box_rows, swizzle128)) return rc;
  std::lock_guard<std::mutex> lock(g_tmap_mu);
  if (g_tmap_cache.size() >= TMAP_CACHE_MAX) g_tmap_cache.clear();  // nobody holds references into it
  g_tmap_cache.emplace(key, *out);
  return Q27B_OK;
}

int q8_tmaps(const void* cache, uint64_t rows, CUtensorMap* vals, CUtensorMap* scales) {
  if (int rc = cached_tmap_2d(vals, cache, rows, AD, AD, 128, 64, true)) return rc;
  return cached_tmap_2d(scales, (const uint8_t*)cache + rows * AD, rows, 16, 16, 16, 64, false);
}

int check_peer_buffer(const void* p, const char* who) {
  int dev = 0;
  Q27B_CK(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(g_peer_mu);
    for (auto& e : g_peer_ok)
      if (e.first == dev && e.second == p) return Q27B_OK;
  }
  cudaPointerAttributes a;
  const cudaError_t pe = cudaPointerGetAttributes(&a, p);
  if (pe != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(Q27B_BAD_SHAPE, std::string(who) + ": exchange buffer is not a CUDA pointer (" + cudaGetErrorString(pe) + ")");
  }
  if (a.type != cudaMemoryTypeDevice) return fail(Q27B_BAD_SHAPE, std::string(who) + ": exchange buffer is not device memory");
  if (a.device != dev) {
    int can = 0;
    Q27B_CK(cudaDeviceCanAccessPeer(&can, dev, a.device));
    if (!can) return fail(Q27B_UNSUPPORTED, std::string(who) + ": no peer access to the device of an exchange buffer");
    const cudaError_t e = cudaDeviceEnablePeerAccess(a.device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
    else Q27B_CK(e);
  }
  std::lock_guard<std::mutex> lock(g_peer_mu);
  if (g_peer_ok.size() < 4096) g_peer_ok.emplace_back(dev, p);
  return Q27B_OK;
}

}  // namespace q27b

using namespace q27b;

extern "C" {

const char* q27b_last_error(void) { return g_err_text(); }

int q27b_attn_workspace_query(uint64_t* decode_bytes, uint64_t* prefill_bytes, uint64_t* paged_bytes, int* fixed) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  if (decode_bytes) *decode_bytes = ctx->dec.floats * sizeof(float);
  if (prefill_bytes) *prefill_bytes = ctx->pf.floats * sizeof(float);
  if (paged_bytes) *paged_bytes = ctx->paged.floats * sizeof(float);
  if (fixed) *fixed = ctx->frozen ? 1 : 0;
  return Q27B_OK;
}

int q27b_attn_workspace_init(uint64_t prefill_bytes, uint64_t paged_bytes) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  if (ctx->frozen) return fail(Q27B_UNSUPPORTED, "attn_workspace_init: already fixed on this device (destroy it first)");
  if (ctx->pf.p && prefill_bytes && prefill_bytes / sizeof(float) != ctx->pf.floats)
    return fail(Q27B_UNSUPPORTED, "attn_workspace_init: the prefill workspace is already allocated at another size");
  if (prefill_bytes) ctx->pf_cap_floats = (size_t)(prefill_bytes / sizeof(float));
  float* dummy;
  size_t cap;
  if (int rc = decode_ws(ctx, &dummy)) return rc;
  if (int rc = prefill_ws(ctx, &dummy, &cap)) return rc;
  if (paged_bytes)
    if (int rc = paged_ws(ctx, (size_t)((paged_bytes + sizeof(float) - 1) / sizeof(float)), &dummy)) return rc;
  ctx->frozen = true;
  return Q27B_OK;
}

int q27b_attn_workspace_destroy(void) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  Q27B_CK(cudaDeviceSynchronize());
  for (WsBuf* b : {&ctx->dec, &ctx->pf, &ctx->paged}) {
    if (b->p) Q27B_CK(cudaFree(b->p));
    b->p = nullptr;
    b->floats = 0;
  }
  if (ctx->ref_scores) Q27B_CK(cudaFree(ctx->ref_scores));
  ctx->ref_scores = nullptr;
  ctx->ref_scores_floats = 0;
  ctx->pf_cap_floats = 0;
  ctx->frozen = false;
  return Q27B_OK;
}

int q27b_device_status(int* status_out) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  int st = 0;
  Q27B_CK(cudaDeviceSynchronize());
  Q27B_CK(cudaMemcpy(&st, ctx->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (st) Q27B_CK(cudaMemset(ctx->status, 0, 256));  // the word, and the tile counters an aborted kernel may have left behind
  int st2 = 0;  // kernels of the no-allocation entry point report into a word of their own
  if (int rc = noalloc_status(ctx->dev, &st2)) return rc;
  st |= st2;
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
  const size_t bytes = (size_t)q27b_xbuf_bytes(nz, rows);
  void* p = nullptr;
  Q27B_CK(cudaMalloc(&p, bytes));  // an allocation of its own: an IPC handle names whole allocations
  Q27B_CK(cudaMemset(p, 0, bytes));
  Q27B_CK(cudaDeviceSynchronize());
  *out = p;
  return Q27B_OK;
}

int q27b_xbuf_reset(void* xbuf, uint64_t bytes, void* stream) {
  if (!xbuf || bytes < 256) return fail(Q27B_BAD_SHAPE, "xbuf_reset: null pointer or less than the header");
  // the step counters of the header, and the data area: a word left over from the broken step carries the tag
  // of a step that the restarted count will reach again
  Q27B_CK(cudaMemsetAsync(xbuf, 0, bytes, (cudaStream_t)stream));
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

// ---- how one sequence / one prefill chunk is shared out over the GPUs of a box (host arithmetic only)
int q27b_plan_single_sequence(int rank, int world, int nkvh, int* kv_head0, int* n_kv_heads, int* z, int* nz) {
  if (world < 1 || rank < 0 || rank >= world || nkvh < 1 || !kv_head0 || !n_kv_heads || !z || !nz)
    return fail(Q27B_BAD_SHAPE, "plan_single_sequence: bad rank / world");
  if (world <= nkvh) {
    if (nkvh % world) return fail(Q27B_BAD_SHAPE, "plan_single_sequence: world must divide the KV heads");
    *n_kv_heads = nkvh / world;
    *kv_head0 = rank * *n_kv_heads;
    *z = 0;
    *nz = 1;
    return Q27B_OK;
  }
  if (world % nkvh) return fail(Q27B_BAD_SHAPE, "plan_single_sequence: world must be a multiple of the KV heads");
  *nz = world / nkvh;
  *kv_head0 = rank / *nz;
  *n_kv_heads = 1;
  *z = rank % *nz;
  return Q27B_OK;
}

int q27b_kv_slice(int n, int z, int nz, int* lo, int* hi) {
  if (n < 0 || nz < 1 || z < 0 || z >= nz || !lo || !hi) return fail(Q27B_BAD_SHAPE, "kv_slice: bad argument");
  int per = (n + nz - 1) / nz;
  per = (per + 63) / 64 * 64;  // slice boundaries are multiples of the 64-position tile
  *lo = std::min(n, z * per);
  *hi = std::min(n, *lo + per);
  return Q27B_OK;
}

int q27b_plan_prefill(int rank, int world, int M, int pos0, int nkvh, int* kv_head0, int* n_kv_heads, int* ranges,
                      int* n_ranges) {
  if (world < 1 || rank < 0 || rank >= world || M < 1 || nkvh < 1 || pos0 < 0 || !kv_head0 || !n_kv_heads || !ranges || !n_ranges)
    return fail(Q27B_BAD_SHAPE, "plan_prefill: bad rank / world / M");
  if (world <= nkvh) {
    if (nkvh % world) return fail(Q27B_BAD_SHAPE, "plan_prefill: world must divide the KV heads");
    *n_kv_heads = nkvh / world;
    *kv_head0 = rank * *n_kv_heads;
    ranges[0] = 0;
    ranges[1] = M;
    *n_ranges = 1;
    return Q27B_OK;
  }
  if (world % nkvh) return fail(Q27B_BAD_SHAPE, "plan_prefill: world must be a multiple of the KV heads");
  const int nq = world / nkvh, s = rank % nq, tiles = (M + 127) / 128, nb = 2 * nq;
  *kv_head0 = rank / nq;
  *n_kv_heads = 1;
  // cost of tile i ~ positions it attends: pos0 + (i + 1) * 128; cuts at equal cumulative cost
  double total = 0;
  for (int i = 0; i < tiles; i++) total += pos0 + std::min(M, (i + 1) * 128);
  std::vector<int> cuts(1, 0);
  double acc = 0;
  int k = 1;
  for (int i = 0; i < tiles; i++) {
    acc += pos0 + std::min(M, (i + 1) * 128);
    while (k < nb && acc >= total * k / nb - 1e-9) {
      cuts.push_back(i + 1);
      k++;
    }
  }
  while ((int)cuts.size() < nb + 1) cuts.push_back(tiles);
  cuts[nb] = tiles;
  auto block = [&](int b, int* a, int* e) {
    *a = std::min(M, cuts[b] * 128);
    *e = std::min(M, cuts[b + 1] * 128);
  };
  int a0, e0, a1, e1;
  block(s, &a0, &e0);
  block(nb - 1 - s, &a1, &e1);
  if (a1 < a0 || (a1 == a0 && e1 < e0)) {
    std::swap(a0, a1);
    std::swap(e0, e1);
  }
  int cnt = 0;
  if (e0 > a0) {
    ranges[0] = a0;
    ranges[1] = e0;
    cnt = 1;
  }
  if (e1 > a1) {
    if (cnt && ranges[1] == a1) ranges[1] = e1;
    else {
      ranges[2 * cnt] = a1;
      ranges[2 * cnt + 1] = e1;
      cnt++;
    }
  }
  *n_ranges = cnt;
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
