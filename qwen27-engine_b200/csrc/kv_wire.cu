// KV rows between the caches and the reference's host ("wire") layout.
//
// The reference moves rows [p0, p1) of a cache to and from host memory (RAM swap of idle slots,
// prompt-cache checkpoints) in this layout per cache: the values [kvh][p1-p0][256 B], then the
// scales [kvh][p1-p0][16 B] (Decoder::kv_copy, src/model.cu:1809-1830). For its contiguous cache
// that is two strided copies. A paged cache (256-position pages behind a page table, which the
// reference does not have) needs a gather / scatter: these kernels pack the rows of one sequence
// from the page pool into a device buffer in exactly that layout (one contiguous copy to pinned
// host memory follows) and unpack it again, so that a slot swapped out by a paged engine can be
// read by the reference's contiguous engine and the other way round.
//
// HBM bound: 272 B read and 272 B written per (KV head, position).
#include "common.cuh"
#include "host.h"

namespace q27b {
namespace {

struct WireParams {
  uint8_t* pool;           // [n_pages][nkvh][256 rows][256 B], then scales [n_pages][nkvh][256][16 B]
  uint8_t* cache;          // or a contiguous cache [nkvh][n_ctx][256 B] + scales (pool == nullptr)
  const int* pages;        // page table row of the sequence: page of positions 256 j .. 256 j + 255
  uint8_t* wire;           // values [nkvh][n][256 B], then scales [nkvh][n][16 B]
  int* status;
  int nkvh, n_pages, n_ctx, p0, n;
};

// One CTA moves the rows of one (KV head, 256-position page) that fall into [p0, p0 + n): on both
// sides they are one contiguous run of values (rows x 256 B) and one of scales (rows x 16 B), so the
// CTA is a plain copy loop with four 16-byte loads in flight per thread.
template <bool TO_WIRE>
__global__ void __launch_bounds__(256) kv_wire_kernel(const WireParams p) {
  pdl_wait();
  pdl_trigger();
  const int kh = blockIdx.y;
  const int pj = p.p0 / Q27B_PAGE + blockIdx.x;                     // page index within the sequence
  const int r0 = max(p.p0, pj * Q27B_PAGE), r1 = min(p.p0 + p.n, (pj + 1) * Q27B_PAGE);
  if (r0 >= r1) return;
  const int rows = r1 - r0, i0 = r0 - p.p0;
  size_t vrow, srow;  // byte offsets of the first row's values and scales on the cache side
  uint8_t* base;
  if (p.pool) {
    const int pg = p.pages[pj];
    if (pg < 0 || pg >= p.n_pages) {  // never touch memory outside the pool: flag it and skip the page
      if (threadIdx.x == 0) atomicOr(p.status, ST_BAD_PAGE);
      return;
    }
    const size_t r = ((size_t)pg * p.nkvh + kh) * Q27B_PAGE + r0 % Q27B_PAGE;
    base = p.pool;
    vrow = r * AD;
    srow = (size_t)p.n_pages * p.nkvh * Q27B_PAGE * AD + r * 16;
  } else {
    const size_t r = (size_t)kh * p.n_ctx + r0;
    base = p.cache;
    vrow = r * AD;
    srow = (size_t)p.nkvh * p.n_ctx * AD + r * 16;
  }
  const size_t wv = ((size_t)kh * p.n + i0) * AD, ws = (size_t)p.nkvh * p.n * AD + ((size_t)kh * p.n + i0) * 16;
  {
    const uint4* src = (const uint4*)(TO_WIRE ? base + vrow : p.wire + wv);
    uint4* dst = (uint4*)(TO_WIRE ? p.wire + wv : base + vrow);
    const int nv = rows * (AD / 16);
    int k = threadIdx.x;
    for (; k + 3 * 256 < nv; k += 4 * 256) {
      const uint4 a = src[k], b = src[k + 256], c = src[k + 512], d = src[k + 768];
      dst[k] = a; dst[k + 256] = b; dst[k + 512] = c; dst[k + 768] = d;
    }
    for (; k < nv; k += 256) dst[k] = src[k];
  }
  {
    const uint4* src = (const uint4*)(TO_WIRE ? base + srow : p.wire + ws);
    uint4* dst = (uint4*)(TO_WIRE ? p.wire + ws : base + srow);
    for (int k = threadIdx.x; k < rows; k += 256) dst[k] = src[k];
  }
}

int launch(const WireParams& p, bool to_wire, cudaStream_t s) {
  const int pages = (p.p0 + p.n - 1) / Q27B_PAGE - p.p0 / Q27B_PAGE + 1;
  const dim3 grid((unsigned)pages, (unsigned)p.nkvh);
  if (to_wire) Q27B_CK(launch_pdl(kv_wire_kernel<true>, grid, dim3(256), 0, s, p));
  else Q27B_CK(launch_pdl(kv_wire_kernel<false>, grid, dim3(256), 0, s, p));
  return Q27B_OK;
}

int check(const void* a, const void* wire, int nkvh, int p0, int p1, const char* who) {
  if (!a || !wire) return fail(Q27B_BAD_SHAPE, std::string(who) + ": null pointer");
  if (nkvh < 1 || nkvh > 65535 || p0 < 0 || p1 <= p0) return fail(Q27B_BAD_SHAPE, std::string(who) + ": bad shape");
  return Q27B_OK;
}

}  // namespace
}  // namespace q27b

using namespace q27b;

extern "C" {

uint64_t q27b_kv_wire_bytes(int nkvh, int n_rows) { return (uint64_t)nkvh * n_rows * (Q27B_HEAD_DIM + 16); }

int q27b_kv_pages_to_wire(const void* pool, const int* pages, void* wire, int nkvh, int n_pages, int p0, int p1,
                          void* stream) {
  if (int rc = check(pool, wire, nkvh, p0, p1, "kv_pages_to_wire")) return rc;
  if (!pages || n_pages < 1) return fail(Q27B_BAD_SHAPE, "kv_pages_to_wire: bad shape");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  WireParams p = {};
  p.pool = (uint8_t*)pool; p.pages = pages; p.wire = (uint8_t*)wire; p.status = ctx->status;
  p.nkvh = nkvh; p.n_pages = n_pages; p.p0 = p0; p.n = p1 - p0;
  return launch(p, true, (cudaStream_t)stream);
}

int q27b_kv_wire_to_pages(void* pool, const int* pages, const void* wire, int nkvh, int n_pages, int p0, int p1,
                          void* stream) {
  if (int rc = check(pool, wire, nkvh, p0, p1, "kv_wire_to_pages")) return rc;
  if (!pages || n_pages < 1) return fail(Q27B_BAD_SHAPE, "kv_wire_to_pages: bad shape");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  WireParams p = {};
  p.pool = (uint8_t*)pool; p.pages = pages; p.wire = (uint8_t*)wire; p.status = ctx->status;
  p.nkvh = nkvh; p.n_pages = n_pages; p.p0 = p0; p.n = p1 - p0;
  return launch(p, false, (cudaStream_t)stream);
}

int q27b_kv_cache_to_wire(const void* cache, void* wire, int nkvh, int n_ctx, int p0, int p1, void* stream) {
  if (int rc = check(cache, wire, nkvh, p0, p1, "kv_cache_to_wire")) return rc;
  if (p1 > n_ctx) return fail(Q27B_BAD_SHAPE, "kv_cache_to_wire: bad shape");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  WireParams p = {};
  p.cache = (uint8_t*)cache; p.wire = (uint8_t*)wire; p.status = ctx->status;
  p.nkvh = nkvh; p.n_ctx = n_ctx; p.p0 = p0; p.n = p1 - p0;
  return launch(p, true, (cudaStream_t)stream);
}

int q27b_kv_wire_to_cache(void* cache, const void* wire, int nkvh, int n_ctx, int p0, int p1, void* stream) {
  if (int rc = check(cache, wire, nkvh, p0, p1, "kv_wire_to_cache")) return rc;
  if (p1 > n_ctx) return fail(Q27B_BAD_SHAPE, "kv_wire_to_cache: bad shape");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  WireParams p = {};
  p.cache = (uint8_t*)cache; p.wire = (uint8_t*)wire; p.status = ctx->status;
  p.nkvh = nkvh; p.n_ctx = n_ctx; p.p0 = p0; p.n = p1 - p0;
  return launch(p, false, (cudaStream_t)stream);
}

}  // extern "C"
