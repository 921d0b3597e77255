// Launcher of the log-sum-exp merge kernel, shared by the decode, prefill and C-ABI entry points.
#pragma once
#include "host.h"

namespace q27b {

struct MergeParams {
  const float* part;    // partials
  int nparts;
  int64_t part_stride;  // generic layout: floats between partials of one row
  int64_t rows;         // output rows
  const float* qg;      // gate source (row r at qg + r*512 + 256) or null
  float* o;             // f32 output [rows][256]
  int8_t* xq;           // q8_1 output instead of o when not null
  float* xd;
  float* part_out;      // when not null: write the merged (M, L, A) [rows][258] and stop
  int T, nqh;           // decode layout only
  const int* seq_len;   // decode layout, batched: sequence s has ceil(seq_len[s] / chunk_len) partials
  int chunk_len;
};

// decode_layout: part is [seq][kvh][chunk][24][258] and rows = seqs * T * nqh.
int launch_merge(const MergeParams& p, bool decode_layout, cudaStream_t s);

}  // namespace q27b
