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

struct DeviceCtx {
  int dev = -1;
  int n_sm = 0;
  int* status = nullptr;      // device status word (see ST_* in common.cuh)
  float* part = nullptr;      // split partials of the decode / prefill kernels
  size_t part_floats = 0;
  int* work = nullptr;        // work list of the batched decode
  size_t work_ints = 0;
  bool decode_attr = false, prefill_attr = false;
  cudaEvent_t split_event = nullptr;  // measurement hook: recorded after the split kernel of a decode call
  unsigned long long* trace = nullptr;  // measurement hook: per-CTA time stamps of the split kernel
};

// Context of the current device, created on first use (allocates the status word).
int device_ctx(DeviceCtx** out);
// Makes ctx->part at least `floats` long (allocates only when it has to grow).
int ensure_part(DeviceCtx* ctx, size_t floats);
int ensure_work(DeviceCtx* ctx, size_t ints);

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

// 2-D byte tensor map over `rows` rows of `row_bytes` bytes (row pitch `pitch_bytes`), copied in
// boxes of box_bytes x box_rows. swizzle128: 128-byte swizzle (box_bytes must then be 128).
// Rows past the end read as zero.
int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint32_t row_bytes, uint64_t pitch_bytes,
                 uint32_t box_bytes, uint32_t box_rows, bool swizzle128);

}  // namespace q27b
