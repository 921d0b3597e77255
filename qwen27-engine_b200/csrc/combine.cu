// Log-sum-exp merge of split partials (m, l, O[256]) -> normalised, gated output.
//
// Replaces attn_combine_kernel (src/attn.cu:294-316) and attn_pf_combine_kernel
// (src/attn.cu:803-822) of the reference: M = max m_c, L = sum l_c e^(m_c - M),
// A = sum O_c e^(m_c - M), y = (A / L) * sigmoid(gate); partials are added in index order, so
// the result does not depend on scheduling. One CTA per output row, one thread per dim; the
// factors e^(m_c - M) are computed once per CTA into shared memory, then every thread streams
// its column of the partials with independent loads. With many partials (one KV head per GPU puts all
// SMs of the GPU on that head: 148 partials per row, and only 24 rows) a row is shared out over several
// CTAs by columns and over thread groups by partials (merge_wide_kernel); where that would be more than one
// wave of CTAs, one CTA of four thread groups that each take a quarter of the partials. Built without fast-math: the q8_1 epilogue
// (q8_store, src/common.cuh:72-81) is specified in IEEE operations.
#include "combine.h"

#include "common.cuh"

#include <cstdlib>

namespace q27b {
namespace {

constexpr int MAX_PARTS = 1024;

// Where row `row` finds its partials and its gate.
struct RowMap {
  const float* first;  // partial 0 of this row
  size_t stride;       // floats between partials
  const float* gate;   // 256 gate values, or null
};

__device__ __forceinline__ RowMap map_generic(const MergeParams& p, int64_t row) {
  return {p.part + row * PROW, (size_t)p.part_stride, p.qg ? p.qg + row * 512 + 256 : nullptr};
}
// Decode layout: part [seq][kvh][chunk][24][258], output row = (seq, t, h), partial row = t*6 + h%6.
__device__ __forceinline__ RowMap map_decode(const MergeParams& p, int64_t row) {
  const int h = (int)(row % p.nqh), t = (int)((row / p.nqh) % p.T);
  const int64_t seq = row / ((int64_t)p.nqh * p.T);
  const int kh = h / GQA, r = t * GQA + h % GQA, nkvh = p.nqh / GQA;
  const float* first = p.part + (((seq * nkvh + kh) * p.nparts) * MAXR + r) * (size_t)PROW;
  return {first, (size_t)MAXR * PROW, p.qg ? p.qg + row * 512 + 256 : nullptr};
}

// Row `row` of slice z in the data area of an exchange buffer (parity = step & 1).
__device__ __forceinline__ uint64_t* xbuf_row(void* xbuf, int parity, int nz, int z, int64_t rows, int64_t row) {
  return (uint64_t*)((uint8_t*)xbuf + XBUF_HEADER_BYTES) + (((size_t)parity * nz + z) * rows + row) * PROW;
}

// XCHG: the push mode of the peer-memory exchange (push_n of MergeParams) is compiled in.
constexpr int MAX_GROUPS = 4;

// NGRP: thread groups of 256 (1, or MAX_GROUPS for many partials).
template <bool DECODE_LAYOUT, bool XCHG, int NGRP>
__global__ void __launch_bounds__(AD * NGRP) merge_kernel(const MergeParams p) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sf[MAX_PARTS];
  __shared__ float sred[32];
  __shared__ float sgl[NGRP], sga[NGRP > 1 ? NGRP - 1 : 1][AD];
  const int64_t row = blockIdx.x;
  constexpr int ngrp = NGRP, nthr = AD * NGRP;
  const int tid = threadIdx.x, grp = tid / AD;
  const int d = tid % AD, lane = tid & 31, warp = tid >> 5;
  RowMap rm = DECODE_LAYOUT ? map_decode(p, row) : map_generic(p, row);
  int np = p.nparts;
  int epoch = 0;
  if (XCHG && p.push_n > 0) epoch = *(volatile int*)p.xbuf;
  if (DECODE_LAYOUT && p.seq_len) {
    const int64_t seq = row / ((int64_t)p.nqh * p.T);
    np = min(np, max(1, (p.seq_len[seq] + p.chunk_len - 1) / p.chunk_len));
  }

  // The first PRE partials of this thread's column (and their sums l) are requested before the
  // maxima are reduced, so that the kernel makes one trip to L2 instead of two.
  constexpr int PRE = NGRP == 1 ? 48 : 16;  // (four groups leave 64 registers per thread)
  // this group's partials [c_lo, c_hi)
  const int per = (np + ngrp - 1) / ngrp, c_lo = min(np, grp * per), c_hi = min(np, c_lo + per);
  const float* col = rm.first + 2 + d;
  float av[PRE], lv[PRE];
#pragma unroll
  for (int c = 0; c < PRE; c++)
    if (c_lo + c < c_hi) {
      av[c] = col[(size_t)(c_lo + c) * rm.stride];
      lv[c] = rm.first[(size_t)(c_lo + c) * rm.stride + 1];
    }
  const float gate = rm.gate ? rm.gate[d] : 0.f;

  // M and the factors
  float mx = M_INIT;
  for (int c = tid; c < np; c += nthr) mx = fmaxf(mx, rm.first[c * rm.stride]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) sred[warp] = mx;
  __syncthreads();
  float M = sred[0];
  for (int i = 1; i < nthr / 32; i++) M = fmaxf(M, sred[i]);
  for (int c = tid; c < np; c += nthr) sf[c] = expf(rm.first[c * rm.stride] - M);
  __syncthreads();

  float L = 0.f, A = 0.f;
#pragma unroll
  for (int c = 0; c < PRE; c++)
    if (c_lo + c < c_hi) {
      const float f = sf[c_lo + c];
      L += lv[c] * f;
      A += av[c] * f;
    }
#pragma unroll 8
  for (int c = c_lo + PRE; c < c_hi; c++) {
    const float f = sf[c];
    L += rm.first[c * rm.stride + 1] * f;
    A += col[c * rm.stride] * f;
  }
  if constexpr (NGRP > 1) {  // add the groups up in group order (group 0 carries on alone)
    if (grp > 0) {
      sga[grp - 1][d] = A;
      if (d == 0) sgl[grp] = L;
    }
    __syncthreads();
    if (grp == 0)
      for (int k = 1; k < ngrp; k++) {
        A += sga[k - 1][d];
        L += sgl[k];
      }
  }
  // Group 0 writes the result; the other groups only keep the CTA's barriers and counters company.
  const bool lead = NGRP == 1 || grp == 0;

  const size_t oi = (size_t)row * AD + d;
  if (XCHG && p.push_n > 0) {  // merged, not normalised, into slot push_z of every rank's exchange buffer
    for (int k = 0; lead && k < p.push_n; k++) {
      uint64_t* po = xbuf_row(p.push_buf[k], epoch & 1, p.push_n, p.push_z, p.rows, row);
      ll_store(po + 2 + d, A, epoch + 1);
      if (d == 0) {
        ll_store(po, M, epoch + 1);
        ll_store(po + 1, L, epoch + 1);
      }
    }
    return;
  }
  if (!lead) return;
  if (p.part_out) {  // merged but not normalised: (M, L, A) for a later merge
    float* po = p.part_out + (size_t)row * PROW;
    po[2 + d] = A;
    if (d == 0) {
      po[0] = M;
      po[1] = L;
    }
    return;
  }
  float y = A / L;
  if (rm.gate) y *= 1.0f / (1.0f + expf(-gate));
  if (!p.xq) {
    p.o[oi] = y;
    return;
  }
  float amax = fabsf(y);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float dd = __fdiv_rn(amax, 127.0f);
  p.xq[oi] = amax == 0.0f ? (int8_t)0 : (int8_t)roundf(__fdiv_rn(y, dd));
  if (lane == 0) p.xd[oi / 32] = __half2float(__float2half_rn(dd));
}

// Many partials per row (one or two KV heads on a whole GPU: 148 or 74 partials per row and few rows): a row is
// shared out over WIDE_SLICES CTAs (4 of 64 dims, or 2 of 128), and inside a CTA of 1024 threads over
// WIDE_GROUPS thread groups (16 or 8) that take every WIDE_GROUPS-th partial: a thread then has at most ten
// loads, all in flight at once, where one CTA per row walks a chain of 37 per thread with a sixth of the SMs.
// Sums are taken in a fixed order (a group's partials in index order, then the groups in order).
constexpr int WIDE_PRE = 10;

template <bool DECODE_LAYOUT, int WIDE_SLICES>
__global__ void __launch_bounds__(1024, 1) merge_wide_kernel(const MergeParams p) {
  constexpr int WIDE_COLS = AD / WIDE_SLICES, WIDE_GROUPS = 1024 / WIDE_COLS;
  pdl_wait();
  pdl_trigger();
  __shared__ float sf[MAX_PARTS];
  __shared__ float sred[32];
  __shared__ float sgl[WIDE_GROUPS], sga[WIDE_GROUPS - 1][WIDE_COLS];
  const int64_t row = blockIdx.x;
  const int slice = blockIdx.y;
  constexpr int nthr = WIDE_COLS * WIDE_GROUPS;
  const int tid = threadIdx.x, grp = tid / WIDE_COLS, dl = tid % WIDE_COLS, d = slice * WIDE_COLS + dl;
  const int lane = tid & 31, warp = tid >> 5;
  const RowMap rm = DECODE_LAYOUT ? map_decode(p, row) : map_generic(p, row);
  int np = p.nparts;
  int epoch = 0;
  if (p.push_n > 0) epoch = *(volatile int*)p.xbuf;
  if (DECODE_LAYOUT && p.seq_len) {
    const int64_t seq = row / ((int64_t)p.nqh * p.T);
    np = min(np, max(1, (p.seq_len[seq] + p.chunk_len - 1) / p.chunk_len));
  }
  // this thread's partials grp, grp + WIDE_GROUPS, ...: the first WIDE_PRE are requested before the maxima
  const float* col = rm.first + 2 + d;
  float av[WIDE_PRE], lv[WIDE_PRE];
#pragma unroll
  for (int k = 0; k < WIDE_PRE; k++) {
    const int c = grp + k * WIDE_GROUPS;
    if (c < np) {
      av[k] = col[(size_t)c * rm.stride];
      lv[k] = rm.first[(size_t)c * rm.stride + 1];
    }
  }
  const float gate = rm.gate ? rm.gate[d] : 0.f;

  float mx = M_INIT;
  for (int c = tid; c < np; c += nthr) mx = fmaxf(mx, rm.first[c * rm.stride]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) sred[warp] = mx;
  __syncthreads();
  float M = sred[0];
#pragma unroll
  for (int i = 1; i < nthr / 32; i++) M = fmaxf(M, sred[i]);
  for (int c = tid; c < np; c += nthr) sf[c] = expf(rm.first[c * rm.stride] - M);
  __syncthreads();

  float L = 0.f, A = 0.f;
#pragma unroll
  for (int k = 0; k < WIDE_PRE; k++) {
    const int c = grp + k * WIDE_GROUPS;
    if (c < np) {
      const float f = sf[c];
      L += lv[k] * f;
      A += av[k] * f;
    }
  }
  for (int c = grp + WIDE_PRE * WIDE_GROUPS; c < np; c += WIDE_GROUPS) {
    const float f = sf[c];
    L += rm.first[c * rm.stride + 1] * f;
    A += col[c * rm.stride] * f;
  }
  if (grp > 0) {
    sga[grp - 1][dl] = A;
    if (dl == 0) sgl[grp] = L;
  }
  __syncthreads();
  const bool lead = grp == 0;
  if (lead)
#pragma unroll
    for (int k = 1; k < WIDE_GROUPS; k++) {
      A += sga[k - 1][dl];
      L += sgl[k];
    }

  if (p.push_n > 0) {  // merged, not normalised, into slot push_z of every rank's exchange buffer
    if (!lead) return;
    const bool fused = p.o != nullptr;  // ... and the final merge of all slices right here, without a second kernel
    for (int k = 0; k < p.push_n; k++) {
      if (fused && k == p.push_z) continue;  // this rank's own slice stays in registers
      uint64_t* po = xbuf_row(p.push_buf[k], epoch & 1, p.push_n, p.push_z, p.rows, row);
      ll_store(po + 2 + d, A, epoch + 1);
      if (dl == 0) {
        ll_store(po, M, epoch + 1);
        ll_store(po + 1, L, epoch + 1);
      }
    }
    if (!fused) return;
    // Every rank has pushed before it waits, so the waits below cannot wait for one another. Same arithmetic,
    // in slice order, as the waiting merge kernel.
    bool ok = true;
    float mz[8], lz[8], az[8];
#pragma unroll
    for (int z = 0; z < 8; z++)
      if (z < p.push_n) {
        if (z == p.push_z) {
          mz[z] = M; lz[z] = L; az[z] = A;
        } else {
          const uint64_t* pz = xbuf_row(p.xbuf, epoch & 1, p.push_n, z, p.rows, row);
          az[z] = ll_load(pz + 2 + d, epoch + 1, ok);
          mz[z] = ll_load(pz, epoch + 1, ok);
          lz[z] = ll_load(pz + 1, epoch + 1, ok);
        }
      }
    if (!ok) {  // a slice never arrived: the status word says so, nothing is written
      if (p.status) atomicOr(p.status, ST_WAIT_EXPIRED);
      return;
    }
    float MM = M_INIT;
#pragma unroll
    for (int z = 0; z < 8; z++)
      if (z < p.push_n) MM = fmaxf(MM, mz[z]);
    float LL = 0.f, AA = 0.f;
#pragma unroll
    for (int z = 0; z < 8; z++)
      if (z < p.push_n) {
        const float f = expf(mz[z] - MM);
        LL += lz[z] * f;
        AA += az[z] * f;
      }
    float y = AA / LL;
    if (rm.gate) y *= 1.0f / (1.0f + expf(-gate));
    p.o[(size_t)row * AD + d] = y;
    if (tid == 0 && atomicAdd(p.xbuf + 2, 1) == (int)p.rows * WIDE_SLICES - 1) {  // the last CTA advances the step
      p.xbuf[2] = 0;
      *(volatile int*)p.xbuf = epoch + 1;
    }
    return;
  }
  if (!lead) return;
  if (p.part_out) {  // merged but not normalised: (M, L, A) for a later merge
    float* po = p.part_out + (size_t)row * PROW;
    po[2 + d] = A;
    if (d == 0) {
      po[0] = M;
      po[1] = L;
    }
    return;
  }
  const size_t oi = (size_t)row * AD + d;
  float y = A / L;
  if (rm.gate) y *= 1.0f / (1.0f + expf(-gate));
  if (!p.xq) {
    p.o[oi] = y;
    return;
  }
  float amax = fabsf(y);  // a warp of the leading group is one q8_1 block of 32 dims
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float dd = __fdiv_rn(amax, 127.0f);
  p.xq[oi] = amax == 0.0f ? (int8_t)0 : (int8_t)roundf(__fdiv_rn(y, dd));
  if (lane == 0) p.xd[oi / 32] = __half2float(__float2half_rn(dd));
}

// The final merge of the peer-memory exchange: one CTA per output row merges the wait_n slices that the ranks
// of the group pushed into this rank's own buffer, waiting (bounded) for each word of the current step; same
// arithmetic, in the same order, as merge_kernel on the gathered partials. The last CTA advances the step.
__global__ void __launch_bounds__(AD, 1) merge_wait_kernel(const MergeParams p) {
  pdl_wait();
  pdl_trigger();
  const int64_t row = blockIdx.x;
  const int d = threadIdx.x, nz = p.wait_n;
  const int epoch = *(volatile int*)p.xbuf;
  bool ok = true;
  float m[8], l[8], a[8];
#pragma unroll
  for (int z = 0; z < 8; z++)
    if (z < nz) {
      const uint64_t* pz = xbuf_row(p.xbuf, epoch & 1, nz, z, p.rows, row);
      a[z] = ll_load(pz + 2 + d, epoch + 1, ok);
      m[z] = ll_load(pz, epoch + 1, ok);
      l[z] = ll_load(pz + 1, epoch + 1, ok);
    }
  const float gate = p.qg ? p.qg[row * 512 + 256 + d] : 0.f;
  if (__syncthreads_or(!ok)) {  // a slice never arrived: the status word says so, nothing is written
    if (d == 0 && p.status) atomicOr(p.status, ST_WAIT_EXPIRED);
    return;
  }
  float M = M_INIT;
#pragma unroll
  for (int z = 0; z < 8; z++)
    if (z < nz) M = fmaxf(M, m[z]);
  float L = 0.f, A = 0.f;
#pragma unroll
  for (int z = 0; z < 8; z++)
    if (z < nz) {
      const float f = expf(m[z] - M);
      L += l[z] * f;
      A += a[z] * f;
    }
  float y = A / L;
  if (p.qg) y *= 1.0f / (1.0f + expf(-gate));
  p.o[(size_t)row * AD + d] = y;
  if (d == 0) {  // the last CTA of the step advances the epoch (nobody reads it again before the next launch)
    if (atomicAdd(p.xbuf + 2, 1) == (int)p.rows - 1) {
      p.xbuf[2] = 0;
      *(volatile int*)p.xbuf = epoch + 1;
    }
  }
}

}  // namespace

int launch_merge(const MergeParams& p, bool decode_layout, cudaStream_t s) {
  if (p.nparts < 1 || p.nparts > MAX_PARTS) return fail(Q27B_BAD_SHAPE, "lse_merge: 1..1024 partials");
  if (p.rows < 1) return Q27B_OK;
  if (p.wait_n > 0) {
    if (p.wait_n > 8 || !p.xbuf || !p.o) return fail(Q27B_BAD_SHAPE, "lse_merge_wait: bad arguments");
    Q27B_CK(launch_pdl(merge_wait_kernel, dim3((unsigned)p.rows), dim3(AD), 0, s, p));
    return Q27B_OK;
  }
  const bool xchg = p.push_n > 0;
  const dim3 grid((unsigned)p.rows);
  // four thread groups once a row has more partials than a 4-head decode call gives it (37 on 148 SMs)
  // (the waiting merge of an exchange has at most 8 partials; the pushing one is a decode-layout merge)
  const bool wide = p.nparts > 64;
  static const bool sliced = [] {  // Q27B_MERGE_SLICED=0: the one-CTA-per-row form for every shape
    const char* e = getenv("Q27B_MERGE_SLICED");
    return !(e && e[0] == '0');
  }();
  // as many slices as keep the CTAs (1024 threads) within one wave of a B200's 148 SMs (with the 96 rows of a
  // 4-head call two slices were measured 3 us slower than one CTA per row, four 6 us)
  const int slices = !(wide && sliced) ? 1 : (p.rows * 4 <= 160 ? 4 : (p.rows * 2 <= 160 ? 2 : 1));
  if (p.push_n > 0 && p.o && slices <= 1) return fail(Q27B_UNSUPPORTED, "fused exchange needs the sliced merge");
  if (slices > 1) {
    const dim3 wgrid((unsigned)p.rows, slices);
    if (decode_layout && slices == 4) Q27B_CK(launch_pdl(merge_wide_kernel<true, 4>, wgrid, dim3(1024), 0, s, p));
    else if (decode_layout) Q27B_CK(launch_pdl(merge_wide_kernel<true, 2>, wgrid, dim3(1024), 0, s, p));
    else if (slices == 4) Q27B_CK(launch_pdl(merge_wide_kernel<false, 4>, wgrid, dim3(1024), 0, s, p));
    else Q27B_CK(launch_pdl(merge_wide_kernel<false, 2>, wgrid, dim3(1024), 0, s, p));
    return Q27B_OK;
  }
  if (decode_layout && xchg && wide) Q27B_CK(launch_pdl(merge_kernel<true, true, MAX_GROUPS>, grid, dim3(AD * MAX_GROUPS), 0, s, p));
  else if (decode_layout && xchg) Q27B_CK(launch_pdl(merge_kernel<true, true, 1>, grid, dim3(AD), 0, s, p));
  else if (decode_layout && wide) Q27B_CK(launch_pdl(merge_kernel<true, false, MAX_GROUPS>, grid, dim3(AD * MAX_GROUPS), 0, s, p));
  else if (decode_layout) Q27B_CK(launch_pdl(merge_kernel<true, false, 1>, grid, dim3(AD), 0, s, p));
  else if (xchg) Q27B_CK(launch_pdl(merge_kernel<false, true, 1>, grid, dim3(AD), 0, s, p));
  else if (wide) Q27B_CK(launch_pdl(merge_kernel<false, false, MAX_GROUPS>, grid, dim3(AD * MAX_GROUPS), 0, s, p));
  else Q27B_CK(launch_pdl(merge_kernel<false, false, 1>, grid, dim3(AD), 0, s, p));
  return Q27B_OK;
}

}  // namespace q27b

using namespace q27b;

extern "C" uint64_t q27b_xbuf_bytes(int nz, int64_t rows) {
  return (uint64_t)XBUF_HEADER_BYTES + 2ull * (uint64_t)nz * (uint64_t)rows * PROW * sizeof(uint64_t);  // {value, tag} words
}

extern "C" int q27b_lse_merge_wait(void* xbuf, int nz, int64_t rows, const float* qg, float* o, void* stream) {
  if (!xbuf || !o) return fail(Q27B_BAD_SHAPE, "lse_merge_wait: null pointer");
  if (nz < 1 || nz > 8 || rows < 1 || rows > 0x7fffffff) return fail(Q27B_BAD_SHAPE, "lse_merge_wait: bad shape");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  MergeParams p = {};
  p.nparts = nz; p.rows = rows; p.qg = qg; p.o = o; p.xbuf = (int*)xbuf; p.wait_n = nz; p.status = ctx->status;
  return launch_merge(p, false, (cudaStream_t)stream);
}

extern "C" int q27b_lse_merge(const float* part, int nparts, int64_t part_stride, int64_t rows, const float* qg, float* o,
                              int8_t* xq, float* xd, void* stream) {
  if (!part || (!o && !xq) || (xq && !xd)) return fail(Q27B_BAD_SHAPE, "lse_merge: null pointer");
  if (rows < 0 || rows > 0x7fffffff || part_stride < 0) return fail(Q27B_BAD_SHAPE, "lse_merge: bad shape");
  MergeParams p = {};
  p.part = part; p.nparts = nparts; p.part_stride = part_stride; p.rows = rows; p.qg = qg; p.o = o; p.xq = xq; p.xd = xd;
  return launch_merge(p, false, (cudaStream_t)stream);
}
