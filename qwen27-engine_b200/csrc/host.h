// Host-side state shared by the entry points: error reporting, the per-device workspace (the
// counterpart of the reference's static AttnWs ws[16], src/attn.cu:869-879) and TMA tensor maps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "../../include/q27b_attn.h"

namespace q27b {

// Records the message for q27b_last_error() and returns `code`.
int fail(int code, const std::string& msg);
void clear_error();
const char* g_err_text();

#define Q27B_CK(x)                                                                                          \
  do {                                                                                                      \
    cudaError_t e_ = (x);                                                                                   \
    if (e_ != cudaSuccess)                                                                                  \
      return ::q27b::fail(Q27B_CUDA_ERROR, std::string(__FILE__) + ":" + std::to_string(__LINE__) + " " #x " -> " + \
                                               cudaGetErrorString(e_));                                    \
  } while (0)

// One per-device workspace buffer. cap_floats > 0: the size it is allocated with on first use and
// never exceeds (a call that would need more fails or splits less).
struct WsBuf {
  float* p = nullptr;
  size_t floats = 0;
};

struct DeviceCtx {
  int dev = -1;
  int n_sm = 0;
  int* status = nullptr;      // device status word (see ST_* in common.cuh) and, from int 16 on, the tile counters
  // Split partials. Three buffers, so that no call frees what another call's captured graph still
  // names (the reference keeps its prefill buffer apart and fixed for the same reason, src/attn.cu:954-959):
  WsBuf dec;                  // decode of one sequence: n_sm chunk partials, fixed size, allocated on first use
  WsBuf pf;                   // prefill: allocated once at pf_cap_floats; the split count is cut to fit
  WsBuf paged;                // batched decode: grows with the batch unless the workspace is frozen
  size_t pf_cap_floats = 0;   // 0: default (see workspace_defaults in host.cu)
  bool frozen = false;        // after q27b_attn_workspace_init: nothing may be allocated any more
  float* ref_scores = nullptr;  // scratch of the slow checking kernel (q27b_attn_decode_ref), grown on demand
  size_t ref_scores_floats = 0;
  bool prefill_attr = false;
  cudaEvent_t split_event = nullptr;  // measurement hook: recorded after the split kernel of a decode call
  cudaEvent_t split_begin = nullptr;  // measurement hook: recorded before it
  bool split_only = false;            // measurement hook: q27b_attn_decode stops after the split kernel
  unsigned long long* trace = nullptr;  // measurement hook: per-CTA time stamps of the split kernel
};

// Context of the current device, created on first use (allocates the status word).
int device_ctx(DeviceCtx** out);
// The decode partial buffer (n_sm chunk partials of 24 x 258 floats), allocated on first use.
int decode_ws(DeviceCtx* ctx, float** out);
// The prefill partial buffer, allocated once at its cap. *max_floats = its size.
int prefill_ws(DeviceCtx* ctx, float** out, size_t* max_floats);
// The batched-decode partial buffer with room for `floats`; grows (free + allocate) when it has to,
// unless the workspace is frozen, in which case a larger request fails with Q27B_UNSUPPORTED.
int paged_ws(DeviceCtx* ctx, size_t floats, float** out);
// Cuts a prefill split plan (ts tiles cut into ns pieces, partial rows Ms * nqh) to what the prefill
// buffer holds: fewer pieces, or no split at all; must_merge (q8_1 through the merge kernel) fails
// instead when not even two pieces fit.
int fit_prefill_split(DeviceCtx* ctx, int* ts, int* ns, int M, int nqh, bool must_merge, float** part);

// True when Q27_PDL=1, the reference's switch with the reference's default (off; src/ops.cu:12-15,
// src/common.cuh:28-42): kernels are then launched with the programmatic-stream-serialization
// attribute, so a kernel's CTAs may be scheduled while its predecessor drains (every kernel here
// begins with griddepcontrol.wait, which holds it until the predecessor has completed and flushed).
// Measured on B200 it does not pay for this pair of kernels (the 226 KB CTAs cannot co-reside).
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// The same through a process-wide cache keyed by every argument and the current device (caches of the
// engine never move, src/model.cu:464-472, so a steady state encodes nothing). The map is copied out:
// a caller never holds a reference into the cache, and the cache may be used from several threads.
int cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint32_t row_bytes, uint64_t pitch_bytes,
                   uint32_t box_bytes, uint32_t box_rows, bool swizzle128);
// Tensor maps of a q8_0 cache of `rows` rows: the int8 values in boxes of 128 bytes x 64 rows with the
// 128-byte swizzle, the f16 scales (behind the values) in boxes of 16 bytes x 64 rows.
int q8_tmaps(const void* cache, uint64_t rows, CUtensorMap* vals, CUtensorMap* scales);
// Status word of q27b_attn_decode_noalloc's kernels on device `dev` (decode.cu), read and cleared.
int noalloc_status(int dev, int* out);
// Checks that kernels of the current device may store into `p` (device memory of this device, or of a
// peer with peer access, which is enabled here once): the exchange buffers of the peer-memory paths.
int check_peer_buffer(const void* p, const char* who);

// 2-D byte tensor map over `rows` rows of `row_bytes` bytes (row pitch `pitch_bytes`), copied in
// boxes of box_bytes x box_rows. swizzle128: 128-byte swizzle (box_bytes must then be 128).
// Rows past the end read as zero.
int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint32_t row_bytes, uint64_t pitch_bytes,
                 uint32_t box_bytes, uint32_t box_rows, bool swizzle128);

}  // namespace q27b
