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
  // Exchange over peer memory (KV-length slices of one sequence on several GPUs). An exchange buffer
  // is [64 ints header][2 parities][nz slices][rows][258 words of 8 bytes: {float value, int step tag}];
  // header: [0] epoch (steps completed), [2] arrival counter of the waiting merge.
  // push_n > 0: the merged (M, L, A) rows go, instead of part_out, into slot push_z of the buffers of
  // all push_n ranks of the group (one 8-byte store per float, tagged epoch + 1; this rank's own buffer
  // included). wait_n > 0: `xbuf` is this rank's own buffer: the kernel waits (bounded) until the words of
  // all wait_n slices carry the tag of the current step, merges them, and the last CTA advances the epoch.
  void* push_buf[8];
  int push_n, push_z;
  int* xbuf;            // this rank's own exchange buffer (push: epoch and counter; wait: everything)
  int wait_n;
  int* status;
};
constexpr int XBUF_HEADER_BYTES = 256;

// decode_layout: part is [seq][kvh][chunk][24][258] and rows = seqs * T * nqh.
int launch_merge(const MergeParams& p, bool decode_layout, cudaStream_t s);

}  // namespace q27b
