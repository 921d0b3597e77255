// Split-K flash-decode over a q8_0 KV cache, warp-specialised: the default decode kernel.
//
// Same operator, same decomposition and same roundings as decode.cu (attn_mma_kernel and the host
// wrapper attn_decode of the reference, src/attn.cu:95-292,894-918; roundings src/attn.cu:10-11):
// one CTA per (position chunk, KV head), 64-position tiles streamed by TMA, S^T = K Q^T and
// O^T += V^T P^T on warp MMAs with the int8 -> f16 conversion in registers, lazily moved reference
// maxima, per-chunk partials (m, l, O) for the log-sum-exp merge kernel.
//
// What differs is who does what. In decode.cu every warp runs both contractions and therefore
// holds the Q fragments (96 registers) and the O accumulators (48) at once: 254 registers per
// thread, two warps per scheduler, and the loop is bound by the latency of its own instruction
// stream (issue slots 39 % busy, DRAM 43 %). Here the two contractions belong to different warps:
//
//   warps 0-3, 4-7    "QK" groups 0 and 1: K tile -> S^T -> P (f16) into shared memory, the row
//                     sums l and the reference maxima m.
//   warps 8-11, 12-15 "PV" groups 0 and 1: V tile and P -> O^T. They own the O accumulators.
//
// QK group g hands its P tiles to PV group g through two P buffers (named barriers: "ready"
// QK -> PV, "free" PV -> QK). Neither kind of warp needs more than 128 registers (the QK warps read
// their Q fragments from shared memory instead of holding them), so sixteen warps fit where eight
// did: four warps per scheduler, twice the latency hiding for the same instruction count.
// K tiles and V tiles have their own rings (3 and 2 deep per group) with their own "full" barriers
// and are refilled by their own consumers (one elected lane each) as soon as the group is provably
// done with a slot, so there is no producer warp and no "empty" barrier.
//
// The query block is staged once per CTA: all threads load Q * kq_scale, round it to f16 and put
// it in shared memory; the QK warps then pick their MMA B fragments from there with two 16-byte
// loads per (row half, position block) (each of the 8 QK warps needs all 24 x 256 values; holding
// them costs 96 registers, loading them from global memory per warp 48 16-byte loads per thread
// before the first MMA).
//
// Which tiles a group takes: a CTA owns the first part of its chunk outright (group g the g-th,
// (g + 2)-th ... tile of it) and, when the launch passes pool counters (p.sched), draws the last
// eighth or so of every chunk of its KV head from a shared pool with one atomicAdd per tile, one
// tile ahead of its use; CTAs that started late or run on a slower SM then take fewer tiles and
// the launch ends evenly. The last CTA to finish resets the counters for the next launch.
//
// The batched decode over pages launches many short CTAs (a chunk of a sequence each, several waves). There
// the kernel runs with ONE tile group per CTA (template parameter NG = 1: 8 warps, half the rings, 109 KB of
// shared memory), two CTAs per SM: the prologue and epilogue of one CTA then overlap the streaming of the
// other, which a single CTA per SM cannot do, and the tail of the launch is half as coarse (config 5 of the
// metric: 2.10 -> 1.95 ms). For a single sequence (one wave of CTAs that start together) the same form was
// measured slower: 296 partials instead of 148 cost the merge more than the split-K kernel gains.
#define Q27B_INLINE_WAITS
#include "common.cuh"
#include "decode_params.h"

#include <mutex>

namespace q27b {
namespace {

constexpr int TILE = 64;                          // positions per tile
constexpr int SEG_BYTES = TILE * 128;             // one 128-byte-wide swizzled box of 64 rows
constexpr int VAL_BYTES = 2 * SEG_BYTES;          // int8 values of a tile (256 B per position)
constexpr int SC_BYTES = TILE * 16;               // f16 scales of a tile (8 per position)
constexpr int HALF_BYTES = VAL_BYTES + SC_BYTES;  // one K (or V) tile with its scales: 17408 = 17 * 1024
constexpr int VDEPTH = 2;                         // V tiles in flight per group
constexpr int KDEPTH = 3;                         // K tiles in flight per group
constexpr int OFF_SC = VAL_BYTES;                 // scales inside a tile buffer
constexpr int P_STRIDE = 36;                      // words per P row (32 position pairs + 4 padding: no bank conflicts)
constexpr int P_WORDS = MAXR * P_STRIDE;
constexpr int Q_STRIDE = 2 * AD + 16;             // bytes per staged Q row (f16; 16 bytes of padding: conflict-free 16-byte reads)
constexpr int SCHED_DONE = 32;                    // p.sched: [KV head] pool counters, [32] CTAs that are done
constexpr float TAU = 8.0f;                       // a score may exceed the reference max by this much
constexpr int O_STRIDE = AD + 4;                  // floats per row of the end-of-kernel O exchange

// Shared memory map of a CTA with NG tile groups (offsets from a 1024-byte aligned base). NG = 2: the
// default, one CTA of 16 warps per SM. NG = 1: 8 warps and half the rings, two CTAs per SM, for launches of
// many short CTAs (the batched decode over pages), where one CTA's prologue and epilogue then overlap the
// other's streaming.
template <int NG>
struct Lay {
  static constexpr int THREADS = 256 * NG;
  static constexpr int OFF_KRING = 0;                                // [KDEPTH][NG groups] K tiles
  static constexpr int OFF_VRING = NG * KDEPTH * HALF_BYTES;         // [VDEPTH][NG groups] V tiles
  static constexpr int RING_BYTES = NG * (KDEPTH + VDEPTH) * HALF_BYTES;
  static constexpr int OFF_Q = RING_BYTES;                           // the staged Q block [24][Q_STRIDE], kept for the whole kernel
  static constexpr int OFF_P = OFF_Q + MAXR * Q_STRIDE;              // [NG groups][2 buffers][24][36] words
  static constexpr int OFF_MAX = OFF_P + NG * 2 * P_WORDS * 4;       // [NG groups][2 buffers][4 warps][24] floats
  static constexpr int OFF_F = OFF_MAX + NG * 2 * 4 * MAXR * 4;      // [NG groups][2 buffers][24] floats: rescale factors for the PV group
  static constexpr int OFF_L = OFF_F + NG * 2 * MAXR * 4;            // [NG groups][4 warps][24] floats: row sums at the end
  static constexpr int OFF_M1 = OFF_L + NG * 4 * MAXR * 4;           // [NG groups][24] floats: reference maxima at the end
  static constexpr int OFF_BAR = OFF_M1 + NG * MAXR * 4;             // fullK[NG * KDEPTH], fullV[NG * VDEPTH]
  static constexpr int OFF_FLAG = OFF_BAR + NG * (KDEPTH + VDEPTH) * 8;
  static constexpr int OFF_TOK = OFF_FLAG + 16;                      // [2 groups][2 buffers] words: "move the maxima" tokens (QK warps)
  static constexpr int OFF_RTOK = OFF_TOK + 16;                      // [2 groups][2 buffers] words: "rescale O" tokens (QK -> PV)
  static constexpr int OFF_SEQ = OFF_RTOK + 16;                      // [2 groups][8] ints: the groups' tile queues
  static constexpr int SMEM_USED = OFF_SEQ + 64;
  static constexpr int SMEM_BYTES = SMEM_USED + 1024;                // slack for the 1024-byte alignment of the ring
  static_assert(OFF_BAR % 8 == 0, "mbarriers are 8-byte aligned");
  static_assert(NG == 1 || MAXR * O_STRIDE * 4 <= RING_BYTES, "O exchange must fit in the ring");
  static_assert(SMEM_BYTES * (3 - NG) + (3 - NG) * 1024 <= 232448, "shared memory of one SM");
};

#ifdef Q27B_WS_PROFILE
constexpr int TRACE_STRIDE = 16;
#else
constexpr int TRACE_STRIDE = 8;
#endif
// Named barriers (0 is __syncthreads).
constexpr int BAR_QK = 1;      // + group: the four QK warps of a group
constexpr int BAR_READY = 3;   // + 2 * group + buffer: P tile written (QK arrives, PV waits)
constexpr int BAR_FREE = 7;    // + 2 * group + buffer: P tile consumed (PV arrives, QK waits)
constexpr int BAR_QKALL = 11;  // all QK warps of the CTA, once, at their end

__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t ldsu16(uint32_t a) {
  uint32_t v;
  asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void stsf(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }
__device__ __forceinline__ float ldsf(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void bar_arrive(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { return __byte_perm(a, b, sel); }

// Row of a 16-row slab that MMA row slot s (0..15) stands for: 8 * (s >> 3) + bitrev3(s & 7).
__device__ __forceinline__ int slot_row(int s) { return (s & 8) | ((s & 1) << 2) | (s & 2) | ((s & 4) >> 2); }
// First of the 4 head dims that k-step ks (0..15) of the S^T MMAs covers for lane quarter tg
// (a 16-byte load is 16 dims = 4 k-steps).
__device__ __forceinline__ int ks_dim0(int ks, int tg) { return 128 * (ks >> 3) + 64 * ((ks >> 2) & 1) + 16 * tg + 4 * (ks & 3); }

// NT = 8-row groups of query rows (ceil(6 T / 8)). PAGED: batched decode over 256-position pages.
template <int NT, bool PAGED, int NG>
__global__ void __launch_bounds__(256 * NG, 3 - NG)
decode_ws_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_ks,
                 const __grid_constant__ CUtensorMap tm_vv, const __grid_constant__ CUtensorMap tm_vs,
                 const DecodeParams p) {
  pdl_wait();
  pdl_trigger();
  using L = Lay<NG>;
  constexpr int WS_THREADS = L::THREADS;
  constexpr int OFF_KRING = L::OFF_KRING, OFF_VRING = L::OFF_VRING, OFF_Q = L::OFF_Q, OFF_P = L::OFF_P, OFF_MAX = L::OFF_MAX,
                OFF_F = L::OFF_F, OFF_L = L::OFF_L, OFF_M1 = L::OFF_M1, OFF_BAR = L::OFF_BAR, OFF_FLAG = L::OFF_FLAG,
                OFF_TOK = L::OFF_TOK, OFF_RTOK = L::OFF_RTOK, OFF_SEQ = L::OFF_SEQ;
  constexpr int PV0 = 128 * NG;  // the first PV thread
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  uint64_t* fullK = (uint64_t*)(sgen + OFF_BAR);
  uint64_t* fullV = fullK + NG * KDEPTH;
  volatile int* abort_flag = (volatile int*)(sgen + OFF_FLAG);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Measurement hook: stamp k of this CTA (see q27b_debug_decode_trace).
  unsigned long long* const trace =
      p.trace ? p.trace + ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * TRACE_STRIDE : nullptr;
  auto stamp = [&](int k) {
    if (trace) trace[k] = global_ns();
  };
  if (tid == 0) stamp(0);
  if (tid == 0) {  // start fetching the tensor maps while the position is being read
    tma_prefetch_desc(&tm_kv);
    tma_prefetch_desc(&tm_vv);
    tma_prefetch_desc(&tm_ks);
    tma_prefetch_desc(&tm_vs);
  }
  const int ch = blockIdx.x, kh = blockIdx.y;
  const int T = p.T, R = GQA * T;
  const int seq = PAGED ? blockIdx.z : 0;
  const float* qn = p.qn + (size_t)seq * T * p.nqh * AD;
  const int g = lane >> 2, tg = lane & 3;

  // The query block: 64 float4 per row, three (six) per thread, requested before anything else waits.
  constexpr int QV = MAXR * 64 / WS_THREADS;
  float4 qv[QV];
#pragma unroll
  for (int j = 0; j < QV; j++) {
    const int i = tid + j * WS_THREADS, r = i >> 6, c4 = i & 63;
    qv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < R) qv[j] = *(const float4*)(qn + ((size_t)(r / GQA) * p.nqh + kh * GQA + r % GQA) * AD + 4 * c4);
  }
  const int pos0 = PAGED ? p.seq_len[seq] - T : *p.pos0;

  // Local rows to attend (n) and the tiles of this CTA. Tiles are numbered over the local rows of the
  // sequence (tile t = rows 64 t ..). A CTA owns the `n_static` tiles from `t_first` on; one sequence
  // (not PAGED) may keep back the tiles from `pool0` on as a pool that the CTAs of the KV head draw
  // from one by one when their own tiles are done (the SMs do not stream at equal rates: with equal
  // static shares the slowest CTA of a 150k-position call ends 5 us after the median one). A CTA
  // folds whatever tiles it gets into one partial: the log-sum-exp merge does not care which.
  int n = pos0 + T - p.base_pos;
  if (p.n_local >= 0) n = min(n, p.n_local);
  n = max(0, min(n, p.n_ctx));
  int t_first, n_static, n_end, pool0, ntiles_all;
  if (PAGED) {
    const int c0 = min(n, ch * p.chunk_len), c1 = min(n, c0 + p.chunk_len);
    t_first = c0 / TILE;
    n_static = (c1 - c0 + TILE - 1) / TILE;
    n_end = c1;
    ntiles_all = pool0 = 0;
  } else {
    ntiles_all = (n + TILE - 1) / TILE;
    const int share = (ntiles_all + p.nch - 1) / p.nch;
    const int own = (p.sched && share > 8) ? share - max(2, share >> 3) - (share >> 4) : share;
    t_first = ch * own;
    n_static = max(0, min(own, ntiles_all - t_first));
    pool0 = p.nch * own;
    n_end = n;
  }
  const bool has_pool = !PAGED && pool0 < ntiles_all;
  float* out = p.part + (((size_t)seq * p.nkvh + kh) * p.nch + ch) * MAXR * PROW;

  if (n_static == 0 && !has_pool) {
    // Nothing to do: neutral partial (src/attn.cu:117-120). The paged merge reads only the chunks
    // that a sequence has, so there nothing is written.
    if (!PAGED)
      for (int i = tid; i < R * PROW; i += WS_THREADS) out[i] = (i % PROW == 0) ? M_INIT : 0.f;
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < NG * (KDEPTH + VDEPTH); s++) mbar_init(&fullK[s], 1);
    *abort_flag = 0;
    for (int i = 0; i < 8; i++) ((volatile uint32_t*)(sgen + OFF_TOK))[i] = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (tid == 0) stamp(1);

  // Row of the K/V tensors at which tile t starts.
  auto tile_row = [&](int t) {
    int row = kh * p.n_ctx + t * TILE;
    if (PAGED) {  // a tile never straddles a page (64 | 256)
      const int pp = t * TILE;
      int pg = p.page_table[(size_t)seq * p.max_pages + pp / Q27B_PAGE];
      if (pg < 0 || pg >= p.n_pages) {  // never read outside the pool: flag it and read page 0
        atomicOr(p.status, ST_BAD_PAGE);
        pg = 0;
      }
      row = (pg * p.nkvh + kh) * Q27B_PAGE + pp % Q27B_PAGE;
    }
    return row;
  };
  const int grp = NG == 2 ? (warp >> 2) & 1 : 0, wq = warp & 3;
  // Tile t into the K (V) buffer that serves the group's j-th tile: buffer 2 (j mod depth) + group.
  auto issue_k = [&](int t, int j) {  // one thread
    const int s = NG * (j % KDEPTH) + grp;
    uint8_t* st = sgen + OFF_KRING + (size_t)s * HALF_BYTES;
    const int row = tile_row(t);
    mbar_expect_tx(&fullK[s], HALF_BYTES);
    tma_load_2d(st, &tm_kv, 0, row, &fullK[s]);
    tma_load_2d(st + SEG_BYTES, &tm_kv, 128, row, &fullK[s]);
    tma_load_2d(st + OFF_SC, &tm_ks, 0, row, &fullK[s]);
  };
  auto issue_v = [&](int t, int j) {  // one thread
    const int s = NG * (j % VDEPTH) + grp;
    uint8_t* st = sgen + OFF_VRING + (size_t)s * HALF_BYTES;
    const int row = tile_row(t);
    mbar_expect_tx(&fullV[s], HALF_BYTES);
    tma_load_2d(st, &tm_vv, 0, row, &fullV[s]);
    tma_load_2d(st + SEG_BYTES, &tm_vv, 128, row, &fullV[s]);
    tma_load_2d(st + OFF_SC, &tm_vs, 0, row, &fullV[s]);
  };
  // The group's j-th tile: its own tiles of the group's parity first, then the pool (-1: no more).
  // Only the loader of a QK group asks; everybody else reads the answer from the queue in shared
  // memory (8 entries per group, entry j mod 8), which the loader fills three tiles ahead.
  auto next_tile = [&](int j) {
    const int i = grp + NG * j;
    if (i < n_static) return t_first + i;
    if (!has_pool) return -1;
    const int t = pool0 + atomicAdd(p.sched + kh, 1);
    return t < ntiles_all ? t : -1;
  };
  const uint32_t sSeq = sbase + OFF_SEQ + grp * 32;

  const bool is_qk = warp < 4 * NG;
  const bool loader = wq == 0 && lane == 0;  // refills this group's K (QK warps) or V (PV warps) halves
  // The ring is started in steps: a request for all six stages of 148 CTAs at once is 30 MB, and the
  // first tile of a CTA then arrives when most of that has been served (3 to 5 us). The first tile
  // of each group is asked for alone, the second a little later, the third when the first has landed.
  int pend = -1;  // QK loader: the tile that goes into the queue next
  if (loader && is_qk) {
    const int t0 = next_tile(0);
    sts32(sSeq + 0, (uint32_t)t0);
    if (t0 >= 0) issue_k(t0, 0);
    const int t1 = t0 < 0 ? -1 : next_tile(1);
    sts32(sSeq + 4, (uint32_t)t1);
    pend = t1 < 0 ? -1 : next_tile(2);
    sts32(sSeq + 8, (uint32_t)pend);
#ifdef Q27B_WS_BURST
    if (t1 >= 0) issue_k(t1, 1);
    if (pend >= 0) issue_k(pend, 2);
#endif
  }

  // Stage the query block: scaled, rounded to f16, [row][256] with padded rows.
  {
    const uint32_t sQ = sbase + OFF_Q;
#pragma unroll
    for (int j = 0; j < QV; j++) {
      const int i = tid + j * WS_THREADS, r = i >> 6, c4 = i & 63;
      if (r < 8 * NT)
        sts64(sQ + r * Q_STRIDE + c4 * 8, pack_h2(qv[j].x * p.kq_scale, qv[j].y * p.kq_scale),
              pack_h2(qv[j].z * p.kq_scale, qv[j].w * p.kq_scale));
    }
  }
  __syncthreads();
  if (loader && !is_qk) {
    const int t0 = (int)lds32(sSeq + 0);
    if (t0 >= 0) issue_v(t0, 0);
#ifdef Q27B_WS_BURST
    const int t1 = (int)lds32(sSeq + 4), t2 = (int)lds32(sSeq + 8);
    if (t1 >= 0) issue_v(t1, 1);
    if (t2 >= 0 && VDEPTH == 3) issue_v(t2, 2);
#endif
  }

  const uint32_t sP = sbase + OFF_P + grp * 2 * P_WORDS * 4;
  const uint32_t sRTok = sbase + OFF_RTOK + grp * 8;
  const uint32_t sF = sbase + OFF_F + grp * 2 * MAXR * 4;
  const uint32_t MAGIC = 0x64646464u;

  if (is_qk) {
    // ======================================================================== QK warps
    // The Q fragments (B operand of S^T = K Q^T) stay in shared memory: k-steps 4hj .. 4hj+3 cover the
    // 16 dims from ks_dim0(4 hj, tg) on of query row 8nt + g, two 16-byte loads.
    const uint32_t sQl = sbase + OFF_Q + g * Q_STRIDE + 32 * tg;
#ifndef Q27B_WS_BURST
    if (loader) {  // the group's second K tile, a little after the first
      const int t1 = (int)lds32(sSeq + 4);
      if (t1 >= 0) issue_k(t1, 1);
    }
#endif
    const int ra = 16 * wq + slot_row(g), rb = ra + 8;  // tile rows of MMA row slots g and g + 8 (S^T)
    // Visible end (local row index, exclusive) of this lane's query rows 8nt + 2tg + e.
    int lim[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int r = 8 * nt + 2 * tg + e;
        lim[nt][e] = min(n_end, pos0 + min(r / GQA, T - 1) + 1 - p.base_pos);
      }
    const int lim_min = min(n_end, pos0 + 1 - p.base_pos);
    float m[NT][2], l[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      m[nt][0] = m[nt][1] = M_INIT;
      l[nt][0] = l[nt][1] = 0.f;
    }
    const uint32_t sMax = sbase + OFF_MAX + grp * 2 * 4 * MAXR * 4;
    const uint32_t sTok = sbase + OFF_TOK + grp * 8;
    const uint32_t sel_sc = (tg & 2) ? 0x3232u : 0x1010u;  // which f16 of a scale word this lane's K blocks use
    // Byte offsets inside a stage that do not depend on the tile. K: chunk tg of rows ra / rb in a
    // segment; chunk 4 + tg is the same address with bit 6 flipped.
    const uint32_t kA = ra * 128 + ((tg ^ (ra & 7)) << 4);
    const uint32_t kB = rb * 128 + ((tg ^ (rb & 7)) << 4);

#ifdef Q27B_WS_PROFILE
    long long w_full = 0, w_free = 0, w_grp = 0, t_a;
#define PROF_BEGIN() t_a = clock64()
#define PROF_END(acc) acc += clock64() - t_a
#else
#define PROF_BEGIN()
#define PROF_END(acc)
#endif
    for (int jt = 0;; jt++) {
      const int tile = (int)lds32(sSeq + (jt & 7) * 4);
      if (tile < 0) break;
      const int s = NG * (jt % KDEPTH) + grp;
      PROF_BEGIN();
      mbar_wait(&fullK[s], (jt / KDEPTH) & 1, abort_flag, p.status);
      PROF_END(w_full);
      if (jt == 0) {
        if (tid == 0) stamp(2);
#ifndef Q27B_WS_BURST
        if (loader && pend >= 0) issue_k(pend, 2);  // the third tile, now that the first has landed
#endif
        if (loader) pend = pend < 0 ? -1 : next_tile(3);
      }
      const uint32_t st = sbase + OFF_KRING + s * HALF_BYTES;
      const int tile_p0 = tile * TILE;
      const bool edge = tile_p0 + TILE > lim_min;  // some row of the tile is masked for some query row

      // ---- S^T = K Q^T for tile rows ra, rb
      // (two accumulator sets, alternating, so that consecutive MMAs do not depend on each other)
      float sacc[NT][4], sacc2[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
        sacc2[nt][0] = sacc2[nt][1] = sacc2[nt][2] = sacc2[nt][3] = 0.f;
      }
      {
        const uint4 sca = lds128(st + OFF_SC + ra * 16), scb = lds128(st + OFF_SC + rb * 16);
        const uint32_t scaw[4] = {sca.x, sca.y, sca.z, sca.w}, scbw[4] = {scb.x, scb.y, scb.z, scb.w};
#pragma unroll
        for (int hj = 0; hj < 4; hj++) {
          const int h = hj >> 1, j = hj & 1;
          const uint4 xa = lds128(st + (kA ^ (j << 6)) + h * SEG_BYTES);  // = swz128(ra, 4j + tg)
          const uint4 xb = lds128(st + (kB ^ (j << 6)) + h * SEG_BYTES);
          const __half2 da = u32_as_h2(prmt(scaw[hj], scaw[hj], sel_sc));
          const __half2 db = u32_as_h2(prmt(scbw[hj], scbw[hj], sel_sc));
          const uint32_t xaw[4] = {xa.x, xa.y, xa.z, xa.w}, xbw[4] = {xb.x, xb.y, xb.z, xb.w};
          uint32_t qw[NT][8];
#pragma unroll
          for (int nt = 0; nt < NT; nt++) {
            const uint4 q0 = lds128(sQl + 8 * nt * Q_STRIDE + 256 * h + 128 * j);
            const uint4 q1 = lds128(sQl + 8 * nt * Q_STRIDE + 256 * h + 128 * j + 16);
            qw[nt][0] = q0.x; qw[nt][1] = q0.y; qw[nt][2] = q0.z; qw[nt][3] = q0.w;
            qw[nt][4] = q1.x; qw[nt][5] = q1.y; qw[nt][6] = q1.z; qw[nt][7] = q1.w;
          }
#pragma unroll
          for (int s2 = 0; s2 < 4; s2++) {
            const uint32_t wa = xaw[s2] ^ 0x80808080u, wb = xbw[s2] ^ 0x80808080u;
            const uint32_t a0 = dq_pair(prmt(wa, MAGIC, 0x4140), da), a2 = dq_pair(prmt(wa, MAGIC, 0x4342), da);
            const uint32_t a1 = dq_pair(prmt(wb, MAGIC, 0x4140), db), a3 = dq_pair(prmt(wb, MAGIC, 0x4342), db);
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
              mma16816((hj & 1) ? sacc2[nt] : sacc[nt], a0, a1, a2, a3, qw[nt][2 * s2], qw[nt][2 * s2 + 1]);
          }
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int c = 0; c < 4; c++) sacc[nt][c] += sacc2[nt][c];
      if (edge) {
        const int pa = tile_p0 + ra, pb = tile_p0 + rb;
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            if (pa >= lim[nt][e]) sacc[nt][e] = -INFINITY;
            if (pb >= lim[nt][e]) sacc[nt][2 + e] = -INFINITY;
          }
      }

      // ---- P = exp(S - m) against the group's reference maxima m. m only moves when some score of
      // the tile exceeds it by more than TAU (and on the group's first tile): then every warp posts
      // its tile maxima, m and l are rescaled, P is recomputed and the PV group is told the factors
      // for O. Otherwise - almost always - a tile costs one group barrier; P stays <= e^TAU, well
      // inside f16.
      const int buf = jt & 1;
      const uint32_t token = (uint32_t)(jt + 1);
      bool exceed = jt == 0;
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++) exceed |= fmaxf(sacc[nt][e], sacc[nt][2 + e]) > m[nt][e] + TAU;
      if (__any_sync(0xffffffffu, exceed) && lane == 0) sts32(sTok + buf * 4, token);
      float lt[NT][2];
      uint32_t pw[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const float mb = m[nt][e] * LOG2E;
          const float pa = ex2(fmaf(sacc[nt][e], LOG2E, -mb)), pb = ex2(fmaf(sacc[nt][2 + e], LOG2E, -mb));
          lt[nt][e] = pa + pb;
          pw[nt][e] = pack_h2(pa, pb);
        }
      // the PV group is done with this P buffer (it held the tile two tiles back)
      PROF_BEGIN();
      if (jt >= 2) bar_sync(BAR_FREE + 2 * grp + buf, 256);
      PROF_END(w_free);
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++)
          // position pair (slot g, slot g + 8) of warp wq = P^T k-slot pair 8wq + g
          sts32(sP + (buf * P_WORDS + (8 * nt + 2 * tg + e) * P_STRIDE + 8 * wq + g) * 4, pw[nt][e]);
      PROF_BEGIN();
      bar_sync(BAR_QK + grp, 128);
      PROF_END(w_grp);
      // All four warps have read the K half of this stage: refill it with the group's tile jt + 3,
      // and ask for the one after that (a pool tile costs a global atomic: its answer is not needed
      // before the next tile's barrier).
      if (loader) {
        sts32(sSeq + ((jt + 3) & 7) * 4, (uint32_t)pend);
        if (pend >= 0) {
          issue_k(pend, jt + 3);
          pend = next_tile(jt + 4);
        }
      }
      if (lds32(sTok + buf * 4) == token) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            float v = fmaxf(sacc[nt][e], sacc[nt][2 + e]);
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
            if (g == 0) stsf(sMax + ((buf * 4 + wq) * MAXR + 8 * nt + 2 * tg + e) * 4, v);
          }
        bar_sync(BAR_QK + grp, 128);
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const int r = 8 * nt + 2 * tg + e;
            float tm = ldsf(sMax + ((buf * 4 + 0) * MAXR + r) * 4);
#pragma unroll
            for (int w = 1; w < 4; w++) tm = fmaxf(tm, ldsf(sMax + ((buf * 4 + w) * MAXR + r) * 4));
            const float mn = fmaxf(m[nt][e], tm);
            const float f = ex2((m[nt][e] - mn) * LOG2E);
            m[nt][e] = mn;
            l[nt][e] *= f;
            if (wq == 0 && g == 0) stsf(sF + (buf * MAXR + r) * 4, f);
            const float mb = mn * LOG2E;
            const float pa = ex2(fmaf(sacc[nt][e], LOG2E, -mb)), pb = ex2(fmaf(sacc[nt][2 + e], LOG2E, -mb));
            lt[nt][e] = pa + pb;
            sts32(sP + (buf * P_WORDS + r * P_STRIDE + 8 * wq + g) * 4, pack_h2(pa, pb));
          }
        if (wq == 0 && lane == 0) sts32(sRTok + buf * 4, token);
        bar_sync(BAR_QK + grp, 128);
      }
      bar_arrive(BAR_READY + 2 * grp + buf, 256);
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        l[nt][0] += lt[nt][0];
        l[nt][1] += lt[nt][1];
      }
    }

    if (lane == 0 && wq == 0) stamp(3 + grp);
#ifdef Q27B_WS_PROFILE
    if (trace && lane == 0 && wq == 1 && grp == 0) {  // cycles this warp spent waiting: K tile, P buffer, its group
      trace[8] = (unsigned long long)w_full;
      trace[9] = (unsigned long long)w_free;
      trace[10] = (unsigned long long)w_grp;
    }
#endif
    // ---- row sums over this warp's positions, and the group's reference maxima
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        float v = l[nt][e];
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        if (g == 0) stsf(sbase + OFF_L + ((grp * 4 + wq) * MAXR + 8 * nt + 2 * tg + e) * 4, v);
        if (wq == 0 && g == 0) stsf(sbase + OFF_M1 + (grp * MAXR + 8 * nt + 2 * tg + e) * 4, m[nt][e]);
      }
    // Both loaders of this CTA have drawn their last pool tile once both Q K^T groups are here. The last CTA
    // of the grid to say so puts the counters back to zero for the next launch. This is done now, while the
    // P V warps are still a tile behind: the fence and the atomic take more than a microsecond, and between
    // the CTA's two barriers below the P V warps would wait for them.
    if (NG == 2) bar_sync(BAR_QKALL, 256);
    if (has_pool && tid == 0) {
      __threadfence();
      const int total = gridDim.x * gridDim.y;
      if (atomicAdd(p.sched + SCHED_DONE, 1) == total - 1) {
        for (int k = 0; k < (int)gridDim.y; k++) p.sched[k] = 0;
        p.sched[SCHED_DONE] = 0;
        __threadfence();
      }
    }
    __syncthreads();  // every tile consumed: the ring is free for the O exchange
    if (NG == 2) __syncthreads();  // (the P V warps' barrier between the two halves of their exchange)
    return;
  }

  // ========================================================================== PV warps
#ifdef Q27B_WS_PROFILE
  long long pv_wfull = 0, pv_wready = 0;
  const long long pv_t0 = clock64();
#endif
  float o[4][NT][4];
#pragma unroll
  for (int mt = 0; mt < 4; mt++)
#pragma unroll
    for (int nt = 0; nt < NT; nt++) o[mt][nt][0] = o[mt][nt][1] = o[mt][nt][2] = o[mt][nt][3] = 0.f;
  {
    // Byte offsets inside a stage that do not depend on the tile. V: 8 bytes of rows slot_row(tg) (+8)
    // and slot_row(tg) + 1 (+8) in this warp's 64-dim quarter; 16 positions further is 2048 bytes
    // further. Scales: this lane's block of those rows.
    const uint32_t vrow = slot_row(tg), vcb = (wq & 1) * 4 + (g >> 1);
    const uint32_t vQ = (wq >> 1) * SEG_BYTES + (g & 1) * 8;
    const uint32_t vA = vQ + vrow * 128 + ((vcb ^ (vrow & 7)) << 4);
    const uint32_t vC = vQ + (vrow + 1) * 128 + ((vcb ^ ((vrow + 1) & 7)) << 4);
    const uint32_t sA = OFF_SC + (2 * wq + (g >> 2)) * 2 + vrow * 16;

    for (int jt = 0;; jt++) {
      const int tile = (int)lds32(sSeq + (jt & 7) * 4);
      if (tile < 0) break;
      const int s = NG * (jt % VDEPTH) + grp;
      const int buf = jt & 1;
      const uint32_t token = (uint32_t)(jt + 1);
      const uint32_t st = sbase + OFF_VRING + s * HALF_BYTES;
      const int tile_p0 = tile * TILE;
      const bool edge = tile_p0 + TILE > n_end;  // rows past the end of the sequence in this tile
#ifndef Q27B_WS_BURST
      if (jt == 0 && loader) {  // the second tile a little after the first
        const int t1 = (int)lds32(sSeq + 4);
        if (t1 >= 0) issue_v(t1, 1);
      }
#endif
#ifdef Q27B_WS_PROFILE
      const long long t_b = clock64();
#endif
      mbar_wait(&fullV[s], (jt / VDEPTH) & 1, abort_flag, p.status);
#ifdef Q27B_WS_PROFILE
      const long long t_c = clock64();
#endif
      bar_sync(BAR_READY + 2 * grp + buf, 256);
#ifdef Q27B_WS_PROFILE
      pv_wfull += t_c - t_b;
      pv_wready += clock64() - t_c;
#endif
      if (jt == 0 && tid == PV0) stamp(5);
      // Every PV warp of the group is past the previous tile: refill its V buffer with the group's
      // tile jt - 1 + VDEPTH (the queue entry was written before the QK group released tile jt - 1).
#ifdef Q27B_WS_BURST
      if (loader && jt >= 1) {
#else
      if (loader && (jt >= 1 || VDEPTH == 3)) {
#endif
        const int jn = jt - 1 + VDEPTH;
        const int tn = (int)lds32(sSeq + (jn & 7) * 4);
        if (tn >= 0) issue_v(tn, jn);
      }
      if (lds32(sRTok + buf * 4) == token) {  // the reference maxima moved: rescale O
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
          for (int e = 0; e < 2; e++) {
            const float f = ldsf(sF + (buf * MAXR + 8 * nt + 2 * tg + e) * 4);
#pragma unroll
            for (int mt = 0; mt < 4; mt++) {
              o[mt][nt][e] *= f;
              o[mt][nt][2 + e] *= f;
            }
          }
      }

      // ---- O^T += V^T P^T for head dims 64wq + 8g .. +7 (8 values of each V row per lane)
      const uint32_t pP = sP + (buf * P_WORDS + g * P_STRIDE + tg) * 4;
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
        const int pa = 16 * ks + slot_row(tg), pb = pa + 8, pc = pa + 1, pd = pa + 9;
        uint32_t b0[NT], b1[NT];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          b0[nt] = lds32(pP + (8 * nt * P_STRIDE + 8 * ks) * 4);
          b1[nt] = lds32(pP + (8 * nt * P_STRIDE + 8 * ks + 4) * 4);
        }
        // rows pa, pb = pa + 8 share one swizzle term, pc = pa + 1, pd = pa + 9 the other
        const uint2 xa = lds64(st + vA + ks * 2048), xb = lds64(st + vA + ks * 2048 + 1024);
        const uint2 xc = lds64(st + vC + ks * 2048), xd = lds64(st + vC + ks * 2048 + 1024);
        uint32_t sa = ldsu16(st + sA + ks * 256), sb = ldsu16(st + sA + ks * 256 + 128);
        uint32_t scc = ldsu16(st + sA + ks * 256 + 16), sd = ldsu16(st + sA + ks * 256 + 144);
        if (edge) {  // rows past the end of the sequence may hold anything: make them exact zeros
          if (tile_p0 + pa >= n_end) sa = 0;
          if (tile_p0 + pb >= n_end) sb = 0;
          if (tile_p0 + pc >= n_end) scc = 0;
          if (tile_p0 + pd >= n_end) sd = 0;
        }
        const __half2 sab = u32_as_h2(prmt(sa, sb, 0x5410)), scd = u32_as_h2(prmt(scc, sd, 0x5410));
        const uint32_t xaw[2] = {xa.x, xa.y}, xbw[2] = {xb.x, xb.y}, xcw[2] = {xc.x, xc.y}, xdw[2] = {xd.x, xd.y};
#pragma unroll
        for (int wi = 0; wi < 2; wi++) {
          const uint32_t ua = xaw[wi] ^ 0x80808080u, ub = xbw[wi] ^ 0x80808080u;
          const uint32_t uc = xcw[wi] ^ 0x80808080u, ud = xdw[wi] ^ 0x80808080u;
          const uint32_t t1 = prmt(ua, ub, 0x5140), t2 = prmt(ua, ub, 0x7362);
          const uint32_t t3 = prmt(uc, ud, 0x5140), t4 = prmt(uc, ud, 0x7362);
          {
            const uint32_t a0 = dq_pair(prmt(t1, MAGIC, 0x4140), sab), a1 = dq_pair(prmt(t1, MAGIC, 0x4342), sab);
            const uint32_t a2 = dq_pair(prmt(t3, MAGIC, 0x4140), scd), a3 = dq_pair(prmt(t3, MAGIC, 0x4342), scd);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) mma16816(o[2 * wi][nt], a0, a1, a2, a3, b0[nt], b1[nt]);
          }
          {
            const uint32_t a0 = dq_pair(prmt(t2, MAGIC, 0x4140), sab), a1 = dq_pair(prmt(t2, MAGIC, 0x4342), sab);
            const uint32_t a2 = dq_pair(prmt(t4, MAGIC, 0x4140), scd), a3 = dq_pair(prmt(t4, MAGIC, 0x4342), scd);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) mma16816(o[2 * wi + 1][nt], a0, a1, a2, a3, b0[nt], b1[nt]);
          }
        }
      }
      // the QK group may overwrite this P buffer (it does so two tiles on, if there are that many)
      if ((int)lds32(sSeq + ((jt + 2) & 7) * 4) >= 0) bar_arrive(BAR_FREE + 2 * grp + buf, 256);
    }
  }
  if (tid == PV0) stamp(6);
#ifdef Q27B_WS_PROFILE
  if (trace && lane == 0 && wq == 1 && grp == 0) {  // cycles this warp spent waiting: V tile, P tile; and in all
    trace[11] = (unsigned long long)pv_wfull;
    trace[12] = (unsigned long long)pv_wready;
    trace[13] = (unsigned long long)(clock64() - pv_t0);
  }
#endif
  __syncthreads();  // every tile consumed: the ring is free for the O exchange; m and l are posted

  if constexpr (NG == 1) {  // one group: its accumulators, maxima and sums are the chunk partial
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int r = 8 * nt + 2 * tg + e;
        if (r >= R) continue;
        float* po = out + (size_t)r * PROW;
#pragma unroll
        for (int mt = 0; mt < 4; mt++) {
          const int d = 64 * wq + 8 * g + 2 * mt;
          *(float2*)(po + 2 + d) = make_float2(o[mt][nt][e], o[mt][nt][2 + e]);
        }
        if (wq == 0 && g == 0) {
          float l0 = 0.f;
#pragma unroll
          for (int w = 0; w < 4; w++) l0 += ldsf(sbase + OFF_L + (w * MAXR + r) * 4);
          po[0] = ldsf(sbase + OFF_M1 + r * 4);
          po[1] = l0;
        }
      }
    if (tid == PV0) stamp(7);
    return;
  }
  // ---- merge the two groups (log-sum-exp) and write the chunk partial
  const uint32_t sO = sbase;
  if (grp == 1) {
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int r = 8 * nt + 2 * tg + e;
#pragma unroll
        for (int mt = 0; mt < 4; mt++) {
          const int d = 64 * wq + 8 * g + 2 * mt;
          stsf(sO + (r * O_STRIDE + d) * 4, o[mt][nt][e]);
          stsf(sO + (r * O_STRIDE + d + 1) * 4, o[mt][nt][2 + e]);
        }
      }
  }
  __syncthreads();
  if (grp == 0) {
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int r = 8 * nt + 2 * tg + e;
        if (r >= R) continue;
        const float m0 = ldsf(sbase + OFF_M1 + r * 4), m1 = ldsf(sbase + OFF_M1 + (MAXR + r) * 4);
        const float M = fmaxf(m0, m1);
        const float f0 = ex2((m0 - M) * LOG2E), f1 = ex2((m1 - M) * LOG2E);
        float* po = out + (size_t)r * PROW;
#pragma unroll
        for (int mt = 0; mt < 4; mt++) {
          const int d = 64 * wq + 8 * g + 2 * mt;
          const float v0 = o[mt][nt][e] * f0 + ldsf(sO + (r * O_STRIDE + d) * 4) * f1;
          const float v1 = o[mt][nt][2 + e] * f0 + ldsf(sO + (r * O_STRIDE + d + 1) * 4) * f1;
          *(float2*)(po + 2 + d) = make_float2(v0, v1);
        }
        if (wq == 0 && g == 0) {
          float l0 = 0.f, l1 = 0.f;
#pragma unroll
          for (int w = 0; w < 4; w++) {
            l0 += ldsf(sbase + OFF_L + (w * MAXR + r) * 4);
            l1 += ldsf(sbase + OFF_L + ((4 + w) * MAXR + r) * 4);
          }
          po[0] = M;
          po[1] = l0 * f0 + l1 * f1;
        }
      }
    if (tid == PV0) stamp(7);
  }
}

template <int NT, int NG>
int launch_ws_nt(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                 const DecodeParams& p, bool paged, int nseq, cudaStream_t s) {
  const dim3 grid(p.nch, p.nkvh, nseq);
  if (paged)
    Q27B_CK(launch_pdl(decode_ws_kernel<NT, true, NG>, grid, dim3(Lay<NG>::THREADS), Lay<NG>::SMEM_BYTES, s, *kv, *ks, *vv, *vs, p));
  else
    Q27B_CK(launch_pdl(decode_ws_kernel<NT, false, NG>, grid, dim3(Lay<NG>::THREADS), Lay<NG>::SMEM_BYTES, s, *kv, *ks, *vv, *vs, p));
  return Q27B_OK;
}

template <int NT, bool PAGED, int NG>
int ws_attr() {
  Q27B_CK(cudaFuncSetAttribute(decode_ws_kernel<NT, PAGED, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay<NG>::SMEM_BYTES));
  if (NG == 1)  // two CTAs per SM need the whole shared-memory carve-out
    Q27B_CK(cudaFuncSetAttribute(decode_ws_kernel<NT, PAGED, NG>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
  return Q27B_OK;
}

}  // namespace

int decode_ws_setup() {
  if (int rc = ws_attr<1, false, 2>()) return rc;
  if (int rc = ws_attr<2, false, 2>()) return rc;
  if (int rc = ws_attr<3, false, 2>()) return rc;
  if (int rc = ws_attr<1, true, 2>()) return rc;
  if (int rc = ws_attr<2, true, 2>()) return rc;
  if (int rc = ws_attr<3, true, 2>()) return rc;
  if (int rc = ws_attr<1, true, 1>()) return rc;
  if (int rc = ws_attr<2, true, 1>()) return rc;
  if (int rc = ws_attr<3, true, 1>()) return rc;
  return Q27B_OK;
}

int launch_decode_ws(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                     const DecodeParams& p, bool paged, int nseq, cudaStream_t s, bool single_group) {
  static bool attr[64] = {};
  static std::mutex attr_mu;
  int dev;
  Q27B_CK(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(attr_mu);
    if (!attr[dev]) {
      if (int rc = decode_ws_setup()) return rc;
      attr[dev] = true;
    }
  }
  const int nt = (GQA * p.T + 7) / 8;
  if (single_group && paged) {  // 8 warps, two CTAs per SM
    if (nt == 1) return launch_ws_nt<1, 1>(kv, ks, vv, vs, p, true, nseq, s);
    if (nt == 2) return launch_ws_nt<2, 1>(kv, ks, vv, vs, p, true, nseq, s);
    return launch_ws_nt<3, 1>(kv, ks, vv, vs, p, true, nseq, s);
  }
  if (nt == 1) return launch_ws_nt<1, 2>(kv, ks, vv, vs, p, paged, nseq, s);
  if (nt == 2) return launch_ws_nt<2, 2>(kv, ks, vv, vs, p, paged, nseq, s);
  return launch_ws_nt<3, 2>(kv, ks, vv, vs, p, paged, nseq, s);
}

}  // namespace q27b
