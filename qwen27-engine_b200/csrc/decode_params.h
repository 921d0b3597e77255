// Parameters shared by the two split-K decode kernels (decode.cu: warp-MMA kernel; decode_tc.cu:
// tcgen05 kernel) and the launcher of the latter.
#pragma once
#include "host.h"

namespace q27b {

struct DecodeParams {
  const float* qn;   // [T][nqh][256]
  float* part;       // [nkvh][nch][24][258]
  const int* pos0;
  int* status;
  int T, nqh, nkvh, n_ctx, nch;
  float kq_scale;
  int base_pos;      // global position of local cache row 0
  int n_local;       // local rows to attend; < 0: all rows up to *pos0 + T
  // paged / batched variant: grid (chunks, nkvh, B), fixed chunk length, rows through the page table
  const int* page_table;  // [B][max_pages]
  const int* seq_len;     // [B], counts the T new tokens
  int max_pages, n_pages, chunk_len;
  // Tile pool of the warp-specialised kernel (one sequence only): [KV head] tiles drawn so far,
  // [32] CTAs that are done; all zero between launches. Null: every CTA keeps to its own share.
  int* sched;
  // measurement hook (null in normal use): [CTA][8] globaltimer stamps of the warp-specialised kernel
  unsigned long long* trace;
};

// Split-K decode over a q8_0 cache on the tcgen05 path (decode_tc.cu). Same grid, same partial
// layout and same tensor maps as the warp-MMA kernel. paged: rows through the page table.
int launch_decode_tc(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                     const DecodeParams& p, bool paged, int nseq, cudaStream_t s);

// The warp-specialised split-K kernel (decode_ws.cu): same grid, partial layout and tensor maps again.
// single_group (paged launches only): CTAs of 8 warps and one tile group, two per SM, instead of 16 warps and two.
int launch_decode_ws(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                     const DecodeParams& p, bool paged, int nseq, cudaStream_t s, bool single_group = false);
// The same with the P V contraction on tcgen05 (decode_wt.cu).
int launch_decode_wt(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                     const DecodeParams& p, bool paged, int nseq, cudaStream_t s);
// Opts the kernels of decode_ws.cu into their shared-memory size on the current device.
int decode_ws_setup();

}  // namespace q27b
