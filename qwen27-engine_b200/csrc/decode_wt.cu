// Split-K flash-decode over a q8_0 KV cache: the warp-specialised kernel of decode_ws.cu with its second
// contraction, O += P V, moved to the 5th-generation tensor cores (tcgen05, accumulator in tensor memory).
// Selectable (q27b_set_decode_kernel(4)); decode_ws.cu stays the default: it is the faster of the two.
//
// Same operator, decomposition, tile schedule and roundings as decode_ws.cu (attn_mma_kernel and the
// host wrapper attn_decode of the reference, src/attn.cu:95-292,894-918; roundings src/attn.cu:10-11).
// What changes is the P V half:
//
//   warps 0-3, 4-7    "QK" groups 0 and 1: K tile -> S^T = K Q^T on warp MMAs with the int8 -> f16 conversion
//                     in registers -> P (f16) into shared memory in the K-major, 128-byte-swizzled layout of a
//                     tcgen05 operand ([query row][64 positions]). They hold the Q fragments in registers (192
//                     registers per thread through setmaxnreg; the converter warps give theirs up: 64) and
//                     refill their own K ring.
//   warps 8-11, 12-15 "CV" groups 0 and 1: V tile -> f16(q * d) into shared memory as the other operand
//                     ([16 positions][256 dims] chunks, dims contiguous, 128-byte swizzle: no transposition,
//                     which the warp-MMA form pays a byte shuffle per value for), one tile per group. One lane
//                     of each group's first converter warp is the group's issuer: it draws the tiles from the
//                     schedule, loads V, and issues the tile's eight tcgen05.mma (O^T[128 dims x 32 rows] +=
//                     V^T[128 x 16 positions] P^T[16 x 32]: the head dims on M, in two halves, the 24 query
//                     rows on N) and their one commit when the QK group has posted the P tile.
//   tensor memory     O^T of group g, half h of the dims: lanes = dims, columns 32 (2 g + h) .. + 31 = rows, f32.
//
// Three things that measurement taught: a tcgen05.mma followed by its own commit costs the issuing thread
// about a thousand cycles, so a tile's MMAs go back to back with one commit; a single thread next to fifteen
// working warps runs at tens of cycles per instruction, so everything serial sits on a converter lane and not
// on the QK warps, which set the pace; and the tensor pipe is shared with the warp MMAs, so the query rows
// belong on N (an eighth of the cost of padding them to M = 128).
// Shared memory pays for the f16 V chunks with shallower rings: two K and two V tiles in flight per group.
//
// The rare rescale of O (the group's reference maxima moved) is done in tensor memory by the QK warps (each
// its 32 lanes) after the MMAs issued so far have completed. Every wait is bounded.
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
constexpr int OFF_SC = VAL_BYTES;                 // scales inside a tile buffer
constexpr int KDEPTH = 2, VDEPTH = 2;             // raw K / V tiles in flight per group
constexpr int NVF = 4;                            // f16 V chunks (16 positions) per group: one tile
constexpr int VF_BYTES = 16 * 2 * AD;             // one chunk: [4 x 64 dims][16 positions][128 B]
constexpr int P_BYTES = MAXR * 128;               // one P tile: 24 rows x 64 positions f16
constexpr int Q_STRIDE = 2 * AD + 16;             // bytes per staged Q row (f16; padding: conflict-free 16-byte reads)
// shared memory map (offsets from a 1024-byte aligned base). The P tiles come first: as the A operand of an
// M = 128 MMA a tile is read 128 rows deep, and the 104 rows behind its 24 must be mapped memory (what they
// hold does not matter: they only reach accumulator rows that nobody reads).
constexpr int OFF_P = 0;                                       // [2 groups][2 buffers] P tiles
constexpr int OFF_VF = OFF_P + 4 * P_BYTES;                    // [2 groups][NVF] f16 V chunks
constexpr int OFF_Q = OFF_VF;                                  // the staged Q block [24][Q_STRIDE]: only until the QK warps hold it in registers
constexpr int OFF_KRING = OFF_VF + 2 * NVF * VF_BYTES;         // [KDEPTH][2 groups] raw K tiles
constexpr int OFF_VRING = OFF_KRING + 2 * KDEPTH * HALF_BYTES; // [VDEPTH][2 groups] raw V tiles
constexpr int OFF_MAX = OFF_VRING + 2 * VDEPTH * HALF_BYTES;   // [2 groups][2 buffers][4 warps][24] floats
constexpr int OFF_F = OFF_MAX + 2 * 2 * 4 * MAXR * 4;          // [2 groups][4 warps][24] floats: rescale factors (a copy per warp)
constexpr int OFF_L = OFF_F + 2 * 4 * MAXR * 4;                    // [2 groups][4 warps][24] floats: row sums at the end
constexpr int OFF_M1 = OFF_L + 2 * 4 * MAXR * 4;               // [2 groups][24] floats: reference maxima at the end
constexpr int OFF_BAR = OFF_M1 + 2 * MAXR * 4;                 // mbarriers, see the enum
constexpr int NBAR = 32;
constexpr int OFF_FLAG = OFF_BAR + NBAR * 8;                   // abort flag, tensor-memory base address
constexpr int OFF_TOK = OFF_FLAG + 16;                         // [2 groups][2 buffers] words: "move the maxima" tokens
constexpr int OFF_SEQ = OFF_TOK + 16;                          // [2 groups][8] ints: the groups' tile queues
constexpr int SMEM_USED = OFF_SEQ + 64;
constexpr int WT_SMEM_BYTES = SMEM_USED + 1024;                // slack for the 1024-byte alignment
constexpr int O_STRIDE = AD + 4;                               // floats per row of the end-of-kernel O exchange
static_assert(MAXR * Q_STRIDE <= 2 * NVF * VF_BYTES, "the staged Q block must fit in the chunks it borrows");
static_assert(OFF_VF % 1024 == 0 && VF_BYTES % 1024 == 0 && P_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
static_assert(OFF_KRING % 1024 == 0 && HALF_BYTES % 1024 == 0, "TMA tiles need 1024-byte alignment");
static_assert(P_BYTES % 1024 == 0 && 32 * 128 <= 2 * P_BYTES, "the B operand is read 32 rows deep: 24 of P and 8 of what follows");
static_assert(2 * MAXR * O_STRIDE * 4 <= 2 * KDEPTH * HALF_BYTES, "O exchange must fit in the K ring");
static_assert(WT_SMEM_BYTES <= 232448, "shared memory budget of one CTA");

// mbarrier indices
enum {
  B_KFULL = 0,                 // [2 * KDEPTH] raw K tile landed (TMA)
  B_VFULL = B_KFULL + 2 * KDEPTH,  // [2 * VDEPTH] raw V tile landed (TMA)
  B_VFFULL = B_VFULL + 2 * VDEPTH, // [2 groups] the tile's f16 V chunks are written (one arrival per converter warp)
  B_PREADY = B_VFFULL + 2,         // [2 groups][2] P tile written by the four QK warps (one arrival, after their barrier)
  B_PFREE = B_PREADY + 4,          // [2 groups][2] the MMAs of a tile have completed: its P tile (two per group,
                                   // alternating) and the group's f16 V chunks are free
  B_ODONE = B_PFREE + 4,           // [2 groups] every MMA of the group has completed
  B_COUNT = B_ODONE + 2,
};
static_assert(B_COUNT <= NBAR, "barrier table");

constexpr float TAU = 8.0f;                           // a score may exceed the reference max by this much
constexpr int WT_THREADS = 512;
// O^T[128 dims x 32 rows] += V^T[128 dims x 16 positions] P^T[16 positions x 32 rows]: f32 += f16 * f16, A (the V
// chunk, dims contiguous) MN-major, B (the P tile, positions contiguous) K-major. With the 24 query rows on
// the N axis an MMA costs an eighth of the 128 x 256 form (query rows on M, padded to 128), which kept the
// tensor pipe, shared with the warp MMAs of the QK warps, busy for a fifth of the time.
constexpr uint32_t IDESC_PV = umma_idesc(1, 0, 0, 1, 0, 128, 32);
constexpr int TMEM_COLS = 128;  // [2 groups][2 halves of the head dims] x 32 columns (query rows); lanes = dims
// Named barriers (0 is __syncthreads).
constexpr int BAR_QK = 1;      // + group: the four QK warps of a group
#ifdef Q27B_WT_PROFILE
constexpr int TRACE_STRIDE = 32;
#else
constexpr int TRACE_STRIDE = 8;
#endif
constexpr int BAR_CV = 3;      // + group: the four converter warps of a group
constexpr int BAR_QREAD = 5;   // the QK warps hold the query block in registers (they arrive, the converter warps wait)
#ifndef Q27B_WT_QK_REGS
#define Q27B_WT_QK_REGS 192
#define Q27B_WT_CV_REGS 64
#endif
constexpr int QK_REGS = Q27B_WT_QK_REGS, CV_REGS = Q27B_WT_CV_REGS;  // registers per thread after the split
static_assert(256 * (QK_REGS + CV_REGS) <= 65536, "the register file of one SM");

template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

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
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory"); }
__device__ __forceinline__ void sts16(uint32_t a, uint32_t v) {
  asm volatile("{ .reg .u16 t; cvt.u16.u32 t, %1; st.shared.u16 [%0], t; }" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void stsf(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }
__device__ __forceinline__ float ldsf(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { return __byte_perm(a, b, sel); }

// O^T[this warp's 32 dims of both halves][row] *= f[row] in tensor memory (f: 24 floats in shared memory).
// Not inlined: the maxima move rarely, and inline the 32 registers of a block would be spilled around in
// the main loop.
__device__ __noinline__ void rescale_cols(uint32_t taddr, uint32_t sf) {
#pragma unroll 1
  for (int h = 0; h < 2; h++) {
    uint32_t v[32];
    tmem_ld32(taddr + h * 32, v);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < MAXR; i++) {
      float f;
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(f) : "r"(sf + 4 * i));
      v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
    }
    tmem_st32(taddr + h * 32, v);
  }
  tc_wait_st();
}

// Row of a 16-row slab that MMA row slot s (0..15) stands for: 8 * (s >> 3) + bitrev3(s & 7).
__device__ __forceinline__ int slot_row(int s) { return (s & 8) | ((s & 1) << 2) | (s & 2) | ((s & 4) >> 2); }

// NT = 8-row groups of query rows (ceil(6 T / 8)). PAGED: batched decode over 256-position pages.
template <int NT, bool PAGED>
__global__ void __launch_bounds__(WT_THREADS, 1)
decode_wt_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_ks,
                 const __grid_constant__ CUtensorMap tm_vv, const __grid_constant__ CUtensorMap tm_vs,
                 const DecodeParams p) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  uint64_t* bar = (uint64_t*)(sgen + OFF_BAR);
  volatile int* abort_flag = (volatile int*)(sgen + OFF_FLAG);
  uint32_t* tmem_slot = (uint32_t*)(sgen + OFF_FLAG + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Measurement hook: stamp k of this CTA (see q27b_debug_decode_trace).
  unsigned long long* const trace =
      p.trace ? p.trace + ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * TRACE_STRIDE : nullptr;
  auto stamp = [&](int k) {
    if (trace) trace[k] = global_ns();
  };
#ifdef Q27B_WT_PROFILE  // more stamps (8..15) and wait-cycle counters (16..23); the trace rows are 32 words then
#define WT_STAMP(cond, k) do { if (cond) stamp(k); } while (0)
#define WT_TIMED(acc, stmt) do { const long long t_ = clock64(); stmt; acc += clock64() - t_; } while (0)
  long long w0 = 0, w1 = 0, w2 = 0, w3 = 0, c0 = 0, c1 = 0, c2 = 0, c3 = 0, tc_ = 0;
#define WT_LAP(acc) do { const long long t_ = clock64(); acc += t_ - tc_; tc_ = t_; } while (0)
#else
#define WT_LAP(acc) do { } while (0)
#define WT_STAMP(cond, k) do { } while (0)
#define WT_TIMED(acc, stmt) do { stmt; } while (0)
#endif
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

  // The query block: 64 float4 per row, three per thread, requested before anything else waits.
  float4 qv[3];
#pragma unroll
  for (int j = 0; j < 3; j++) {
    const int i = tid + j * WT_THREADS, r = i >> 6, c4 = i & 63;
    qv[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < R) qv[j] = *(const float4*)(qn + ((size_t)(r / GQA) * p.nqh + kh * GQA + r % GQA) * AD + 4 * c4);
  }
  const int pos0 = PAGED ? p.seq_len[seq] - T : *p.pos0;

  // Local rows to attend (n) and the tiles of this CTA: the schedule of decode_ws.cu (own tiles, then the
  // pool of the KV head).
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
      for (int i = tid; i < R * PROW; i += WT_THREADS) out[i] = (i % PROW == 0) ? M_INIT : 0.f;
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < 2 * (KDEPTH + VDEPTH); s++) mbar_init(&bar[B_KFULL + s], 1);
    mbar_init(&bar[B_VFFULL], 4);
    mbar_init(&bar[B_VFFULL + 1], 4);
    for (int s = 0; s < 4; s++) {
      mbar_init(&bar[B_PREADY + s], 1);
      mbar_init(&bar[B_PFREE + s], 1);
    }
    mbar_init(&bar[B_ODONE], 1);
    mbar_init(&bar[B_ODONE + 1], 1);
    *abort_flag = 0;
    for (int i = 0; i < 4; i++) ((volatile uint32_t*)(sgen + OFF_TOK))[i] = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
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
  const int grp = (warp >> 2) & 1, wq = warp & 3;
  // Tile t into the raw K (V) buffer that serves the group's j-th tile: buffer 2 (j mod depth) + group.
  auto issue_k = [&](int t, int j) {  // one thread
    const int s = 2 * (j % KDEPTH) + grp;
    uint8_t* st = sgen + OFF_KRING + (size_t)s * HALF_BYTES;
    const int row = tile_row(t);
    mbar_expect_tx(&bar[B_KFULL + s], HALF_BYTES);
    tma_load_2d(st, &tm_kv, 0, row, &bar[B_KFULL + s]);
    tma_load_2d(st + SEG_BYTES, &tm_kv, 128, row, &bar[B_KFULL + s]);
    tma_load_2d(st + OFF_SC, &tm_ks, 0, row, &bar[B_KFULL + s]);
  };
  auto issue_v = [&](int t, int j) {  // one thread
    const int s = 2 * (j % VDEPTH) + grp;
    uint8_t* st = sgen + OFF_VRING + (size_t)s * HALF_BYTES;
    const int row = tile_row(t);
    mbar_expect_tx(&bar[B_VFULL + s], HALF_BYTES);
    tma_load_2d(st, &tm_vv, 0, row, &bar[B_VFULL + s]);
    tma_load_2d(st + SEG_BYTES, &tm_vv, 128, row, &bar[B_VFULL + s]);
    tma_load_2d(st + OFF_SC, &tm_vs, 0, row, &bar[B_VFULL + s]);
  };
  // The group's j-th tile: its own tiles of the group's parity first, then the pool (-1: no more).
  // Only the group's issuing lane (below) asks; everybody else reads the answer from the queue in
  // shared memory (8 entries per group, entry j mod 8), which that lane fills four tiles ahead: entry
  // j + 4 before it commits the MMAs of tile j. Whoever reads entry j + 2 or an earlier one has waited
  // for the MMAs of tile j - 2 or later before.
  // Asking and using are apart: a pool tile costs an atomic on global memory, whose answer the issuing lane
  // only looks at one tile later (tile_of), so that it never waits for it.
  const int t_limit = PAGED ? t_first + n_static : ntiles_all;
  auto ask_tile = [&](int j) {
    const int i = grp + 2 * j;
    if (i < n_static) return t_first + i;
    if (!has_pool) return 0x7fffffff;
    return pool0 + atomicAdd(p.sched + kh, 1);
  };
  auto tile_of = [&](int asked) { return asked < t_limit ? asked : -1; };
  const uint32_t sSeq = sbase + OFF_SEQ + grp * 32;

  const bool is_qk = warp < 8;
  // One lane per group (of its first converter warp) does what is serial: it asks for tiles, issues the V
  // loads and the tcgen05 MMAs. A single thread next to fifteen working warps is slow (tens of cycles per
  // instruction), so the QK warps, which set the pace, keep only the refill of their own K ring.
  const bool issuer = !is_qk && wq == 0 && lane == 0;
  // issuer: the group's tiles j + 2, j + 3 and j + 4, and what it asked for j + 5
  int e2 = -1, e3 = -1, e4 = -1, asked = 0x7fffffff;
  if (issuer) {
    const int t0 = tile_of(ask_tile(0));
    sts32(sSeq + 0, (uint32_t)t0);
    if (t0 >= 0) issue_k(t0, 0), issue_v(t0, 0);
    const int t1 = t0 < 0 ? -1 : tile_of(ask_tile(1));
    sts32(sSeq + 4, (uint32_t)t1);
    if (t1 >= 0) issue_k(t1, 1), issue_v(t1, 1);
    e2 = t1 < 0 ? -1 : tile_of(ask_tile(2));
    sts32(sSeq + 8, (uint32_t)e2);
    e3 = e2 < 0 ? -1 : tile_of(ask_tile(3));
    sts32(sSeq + 12, (uint32_t)e3);
    e4 = e3 < 0 ? -1 : tile_of(ask_tile(4));
    if (e4 >= 0) asked = ask_tile(5);
  }

  // Stage the query block: scaled, rounded to f16, [row][256] with padded rows.
  {
    const uint32_t sQ = sbase + OFF_Q;
#pragma unroll
    for (int j = 0; j < 3; j++) {
      const int i = tid + j * WT_THREADS, r = i >> 6, c4 = i & 63;
      if (r < 8 * NT)
        sts64(sQ + r * Q_STRIDE + c4 * 8, pack_h2(qv[j].x * p.kq_scale, qv[j].y * p.kq_scale),
              pack_h2(qv[j].z * p.kq_scale, qv[j].w * p.kq_scale));
    }
  }
  __syncthreads();
  const uint32_t MAGIC = 0x64646464u;

  if (is_qk) {
    // ======================================================================== QK warps
    reg_inc<QK_REGS>();
    // The B fragments of Q^T for all 16 k-steps: lane (g, tg) holds dims 64 hj + 16 tg .. + 15 of rows 8 nt + g.
    uint32_t qreg[NT][32];
    {
      const uint32_t sQl = sbase + OFF_Q + g * Q_STRIDE + 32 * tg;
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int hj = 0; hj < 4; hj++) {
          const uint4 q0 = lds128(sQl + 8 * nt * Q_STRIDE + 128 * hj), q1 = lds128(sQl + 8 * nt * Q_STRIDE + 128 * hj + 16);
          qreg[nt][8 * hj + 0] = q0.x; qreg[nt][8 * hj + 1] = q0.y; qreg[nt][8 * hj + 2] = q0.z; qreg[nt][8 * hj + 3] = q0.w;
          qreg[nt][8 * hj + 4] = q1.x; qreg[nt][8 * hj + 5] = q1.y; qreg[nt][8 * hj + 6] = q1.z; qreg[nt][8 * hj + 7] = q1.w;
        }
      asm volatile("bar.arrive %0, %1;" ::"r"(BAR_QREAD), "r"(WT_THREADS) : "memory");
    }
    const uint32_t sPg = sbase + OFF_P + grp * 2 * P_BYTES;
    const uint32_t sF = sbase + OFF_F + (grp * 4 + wq) * MAXR * 4;  // this warp's copy of the rescale factors
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
    // Byte offsets inside a raw tile that do not depend on the tile. K: chunk tg of rows ra / rb in a
    // segment; chunk 4 + tg is the same address with bit 6 flipped.
    const uint32_t kA = ra * 128 + ((tg ^ (ra & 7)) << 4);
    const uint32_t kB = rb * 128 + ((tg ^ (rb & 7)) << 4);
    // Where this lane's P values go: positions ra (8-position chunk 2 wq, slot slot_row(g)) and rb (chunk
    // 2 wq + 1) of query row r; the chunk index is XORed with r & 7 (128-byte swizzle).
    // (r & 7 = 2 tg + e whatever nt is, so the two offsets below serve all rows: + 1024 nt; the second chunk is
    // the same address with bit 4 flipped)
    const uint32_t pofs0 = (2 * tg) * 128 + (((2 * wq) ^ (2 * tg)) << 4) + slot_row(g) * 2;
    const uint32_t pofs1 = (2 * tg + 1) * 128 + (((2 * wq) ^ (2 * tg + 1)) << 4) + slot_row(g) * 2;

    for (int jt = 0;; jt++) {
      const int tile = (int)lds32(sSeq + (jt & 7) * 4);
      if (tile < 0) break;
      const int s = 2 * (jt % KDEPTH) + grp;
      WT_TIMED(w0, mbar_wait(&bar[B_KFULL + s], (jt / KDEPTH) & 1, abort_flag, p.status));
      if (jt == 0 && tid == 0) stamp(2);
#ifdef Q27B_WT_PROFILE
      tc_ = clock64();
#endif
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
#pragma unroll
          for (int s2 = 0; s2 < 4; s2++) {
            const uint32_t wa = xaw[s2] ^ 0x80808080u, wb = xbw[s2] ^ 0x80808080u;
            const uint32_t a0 = dq_pair(prmt(wa, MAGIC, 0x4140), da), a2 = dq_pair(prmt(wa, MAGIC, 0x4342), da);
            const uint32_t a1 = dq_pair(prmt(wb, MAGIC, 0x4140), db), a3 = dq_pair(prmt(wb, MAGIC, 0x4342), db);
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
              mma16816((hj & 1) ? sacc2[nt] : sacc[nt], a0, a1, a2, a3, qreg[nt][8 * hj + 2 * s2], qreg[nt][8 * hj + 2 * s2 + 1]);
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

      // ---- P = exp(S - m) against the group's reference maxima m (they move only when a score exceeds
      // them by more than TAU, and on the group's first tile)
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
      // the MMAs that read this P buffer two tiles back have completed
      WT_STAMP(jt == 0 && tid == 0, 10);
      WT_LAP(c0);  // S and exp
      if (jt >= 2) WT_TIMED(w1, mbar_wait(&bar[B_PFREE + 2 * grp + buf], ((jt >> 1) - 1) & 1, abort_flag, p.status));
      const uint32_t sPt = sPg + buf * P_BYTES;
      const uint32_t pst[2] = {sPt + pofs0, sPt + pofs1};
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          sts16(pst[e] + 1024 * nt, pw[nt][e] & 0xffffu);
          sts16((pst[e] ^ 16u) + 1024 * nt, pw[nt][e] >> 16);
        }
      WT_LAP(c1);  // free P tile, P stores
      fence_proxy_async();  // the tile is read by the tensor core
      WT_LAP(c2);  // the fence
      WT_TIMED(w2, bar_sync(BAR_QK + grp, 128));
#ifdef Q27B_WT_PROFILE
      tc_ = clock64();
#endif
      // All four warps have read this raw K tile: it takes the group's tile jt + 2.
      if (wq == 0 && lane == 0) {
        const int tn = (int)lds32(sSeq + ((jt + 2) & 7) * 4);
        if (tn >= 0) issue_k(tn, jt + 2);
      }
      const bool moved = lds32(sTok + buf * 4) == token;
      if (moved) {
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
            if (g == 0) stsf(sF + r * 4, f);
            const float mb = mn * LOG2E;
            const float pa = ex2(fmaf(sacc[nt][e], LOG2E, -mb)), pb = ex2(fmaf(sacc[nt][2 + e], LOG2E, -mb));
            lt[nt][e] = pa + pb;
            sts16(pst[e] + 1024 * nt, pack_h2(pa, pb) & 0xffffu);
            sts16((pst[e] ^ 16u) + 1024 * nt, pack_h2(pa, pb) >> 16);
          }
        fence_proxy_async();
        if (jt > 0) {
          // O of this group holds the tiles before jt, scaled to the old maxima: once the MMAs of the
          // previous tile have completed, every warp of the group multiplies the 32 dims (lanes of tensor
          // memory) that it may touch, all rows.
          __syncwarp();  // this warp's factors are in shared memory
          mbar_wait(&bar[B_PFREE + 2 * grp + (buf ^ 1)], ((jt - 1) >> 1) & 1, abort_flag, p.status);
          tc_fence_after();
          rescale_cols(tmem + ((uint32_t)(32 * wq) << 16) + grp * 64, sF);
          tc_fence_before();
        }
        bar_sync(BAR_QK + grp, 128);
      }
      // Every warp of the group is past its barrier: the P tile is complete and fenced, the raw K tile read.
      if (wq == 0 && lane == 0) mbar_arrive(&bar[B_PREADY + 2 * grp + buf]);
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        l[nt][0] += lt[nt][0];
        l[nt][1] += lt[nt][1];
      }
      WT_LAP(c3);  // after the group barrier
    }
    if (tid == 0) stamp(4);
#ifdef Q27B_WT_PROFILE
    if (trace && tid == 32) {  // one QK warp: cycles waiting for K tiles, free P tiles, its group; and working
      trace[16] = (unsigned long long)w0;
      trace[17] = (unsigned long long)w1;
      trace[18] = (unsigned long long)w2;
      trace[28] = (unsigned long long)c0;
      trace[29] = (unsigned long long)c1;
      trace[30] = (unsigned long long)c2;
      trace[31] = (unsigned long long)c3;
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
    reg_dec<128>();
  } else {
    // ======================================================================== converter warps
    // V: 64 rows x 16 chunks of 16 int8 -> 16 f16 (one rounding of q * d, as src/attn.cu:59-76), 16 positions
    // (one MMA k-step) at a time. Item = (row, 16-dim chunk); eight neighbouring lanes take 4 chunks of rows
    // rho and rho ^ 5, which keeps the swizzled 16-byte loads and the swizzled 16-byte stores conflict-free.
    // A thread owns the same chunk of rows row0 and row0 + 8 of every 16 positions.
    const int ct = tid - 256 - grp * 128;
    const int cv_row0 = (2 * (ct >> 5)) ^ (5 * ((ct >> 2) & 1)), cv_c16 = (ct & 3) + 4 * ((ct >> 3) & 3);
    const uint32_t cv_src = (cv_c16 >> 3) * SEG_BYTES + swz128(cv_row0, cv_c16 & 7);
    const uint32_t cv_sc = OFF_SC + cv_row0 * 16 + (cv_c16 >> 1) * 2;
    const uint32_t cv_dst = (cv_c16 >> 2) * (16 * 128) + swz128(cv_row0, 2 * (cv_c16 & 3));
    reg_dec<CV_REGS>();
    bar_sync(BAR_QREAD, WT_THREADS);  // the chunks' memory held the staged query block until here
    WT_STAMP(tid == 256, 13);
#ifdef Q27B_WT_PROFILE
    const long long cv_t0 = clock64();
#endif
    for (int jt = 0;; jt++) {
      const int tile = (int)lds32(sSeq + (jt & 7) * 4);
      if (tile < 0) break;
      const int s = 2 * (jt % VDEPTH) + grp, buf = jt & 1;
      const uint32_t st = sbase + OFF_VRING + s * HALF_BYTES;
      const int tile_p0 = tile * TILE;
      WT_TIMED(w0, mbar_wait(&bar[B_VFULL + s], (jt / VDEPTH) & 1, abort_flag, p.status));
      WT_STAMP(jt == 0 && tid == 256, 8);
      // The MMAs of the group's previous tile have read the chunks. A long wait next to working warps: one
      // warp polls the barrier, the others sleep at a hardware barrier until it has seen the phase.
      if (jt >= 1) {
        if (wq == 0) WT_TIMED(w1, mbar_wait(&bar[B_PFREE + 2 * grp + (buf ^ 1)], ((jt - 1) >> 1) & 1, abort_flag, p.status));
        WT_TIMED(w1, bar_sync(BAR_CV + grp, 128));
      }
#pragma unroll
      for (int kh2 = 0; kh2 < 2; kh2++) {  // two chunks at a time: their eight loads are in flight together
        uint4 x[4];
        uint32_t d[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          x[k] = lds128(st + cv_src + (4 * kh2 + k) * 1024);
          d[k] = ldsu16(st + cv_sc + (4 * kh2 + k) * 128);
        }
        if (tile_p0 + TILE > n_end) {  // (the last tile only)
          // rows past the end of the sequence may hold anything: P is 0 there, V must be too
#pragma unroll
          for (int k = 0; k < 4; k++)
            if (tile_p0 + 32 * kh2 + 8 * k + cv_row0 >= n_end) d[k] = 0, x[k] = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const __half2 dd = u32_as_h2(prmt(d[k], d[k], 0x1010));
          const uint32_t xw[4] = {x[k].x ^ 0x80808080u, x[k].y ^ 0x80808080u, x[k].z ^ 0x80808080u, x[k].w ^ 0x80808080u};
          uint32_t o[8];
#pragma unroll
          for (int w = 0; w < 4; w++) {
            o[2 * w] = dq_pair(prmt(xw[w], MAGIC, 0x4140), dd);
            o[2 * w + 1] = dq_pair(prmt(xw[w], MAGIC, 0x4342), dd);
          }
          const uint32_t dst = sbase + OFF_VF + (grp * NVF + 2 * kh2 + (k >> 1)) * VF_BYTES + cv_dst + (k & 1) * 1024;
          sts128(dst, o[0], o[1], o[2], o[3]);
          sts128(dst ^ 16u, o[4], o[5], o[6], o[7]);
        }
      }
      fence_proxy_async();  // the chunks are read by the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_VFFULL + grp]);
      WT_STAMP(jt == 0 && tid == 256, 9);
      if (issuer) {
        // All four converter warps are done with this raw V tile and have written its chunks.
        WT_TIMED(w2, mbar_wait(&bar[B_VFFULL + grp], jt & 1, abort_flag, p.status));
        if (e2 >= 0) issue_v(e2, jt + 2);
        sts32(sSeq + ((jt + 4) & 7) * 4, (uint32_t)e4);  // before the commit below: see the queue's rule
        // ---- the tile's eight MMAs (four 16-position steps x two halves of the dims), back to back and one
        // commit (an MMA followed by its own commit costs the issuing thread about a thousand cycles)
        WT_TIMED(w3, mbar_wait(&bar[B_PREADY + 2 * grp + buf], (jt >> 1) & 1, abort_flag, p.status));
        tc_fence_after();
        if (!*abort_flag) {
          const uint32_t sPt = sbase + OFF_P + (grp * 2 + buf) * P_BYTES;
#pragma unroll
          for (int kk = 0; kk < 4; kk++) {
            const uint64_t db = umma_desc_sw128(sPt + kk * 32, 16, 1024);
#pragma unroll
            for (int h = 0; h < 2; h++) {  // dims 128 h .. + 127: two 64-dim blocks of the chunk
              const uint64_t da = umma_desc_sw128(sbase + OFF_VF + (grp * NVF + kk) * VF_BYTES + h * 2 * 16 * 128, 16 * 128, 1024);
              tc_mma_f16(tmem + (grp * 2 + h) * 32, da, db, IDESC_PV, (jt > 0 || kk > 0) ? 1u : 0u);
            }
          }
          tc_commit(&bar[B_PFREE + 2 * grp + buf]);
        }
        if (jt == 0 && tid == 256) stamp(3);
        e2 = e3;
        e3 = e4;
        if (e4 >= 0) {
          e4 = tile_of(asked);  // asked for one tile ago
          if (e4 >= 0) asked = ask_tile(jt + 6);
        }
      }
    }
    if (issuer) tc_commit(&bar[B_ODONE + grp]);
#ifdef Q27B_WT_PROFILE
    if (trace && tid == 256) {  // the issuing lane: cycles waiting for the other converter warps, for P
      trace[20] = (unsigned long long)w2;
      trace[21] = (unsigned long long)w3;
    }
    if (trace && tid == 288) {  // a converter warp that does not issue: cycles waiting for V tiles, free chunks; in all
      trace[22] = (unsigned long long)w0;
      trace[23] = (unsigned long long)w1;
      trace[24] = (unsigned long long)(clock64() - cv_t0);
    }
#endif
    reg_inc<128>();
    WT_STAMP(tid == 256, 15);
  }
  __syncthreads();  // every tile consumed: the rings are free for the O exchange; m and l are posted
  WT_STAMP(tid == 0, 12);

  // ---- O^T out of tensor memory: lanes = dims, columns = rows. Warp w may read lanes 32 (w mod 4) .. + 31; it
  // takes them from half (w / 4) mod 2 of group w / 8, scales each row to the common maxima of the two groups
  // and puts it into shared memory as [group][row][dim].
  const uint32_t sO = sbase + OFF_KRING;  // f32 [2 groups][24][O_STRIDE]
  {
    const int og = warp >> 3, oh = (warp >> 2) & 1;
    mbar_wait(&bar[B_ODONE + og], 0, abort_flag, p.status);
    tc_fence_after();
    if (tid == 0) stamp(5);
    uint32_t v[32];
    tmem_ld32(tmem + ((uint32_t)(32 * wq) << 16) + (og * 2 + oh) * 32, v);
    tc_wait_ld();
    const int dim = oh * 128 + wq * 32 + lane;
#pragma unroll
    for (int i = 0; i < MAXR; i++) {
      if (i < R) {
        const float m0 = ldsf(sbase + OFF_M1 + i * 4), m1 = ldsf(sbase + OFF_M1 + (MAXR + i) * 4);
        const float mg = og ? m1 : m0;
        // a group without tiles never issued an MMA: its accumulator is not initialised
        const float x = mg <= M_INIT ? 0.f : __uint_as_float(v[i]) * ex2((mg - fmaxf(m0, m1)) * LOG2E);
        stsf(sO + ((og * MAXR + i) * O_STRIDE + dim) * 4, x);
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (tid == 0) stamp(6);
  // all threads: the chunk partial = the two groups added up
  for (int i = tid; i < R * (AD / 4); i += WT_THREADS) {
    const int r = i / (AD / 4), c4 = i % (AD / 4);
    const uint4 a = lds128(sO + (r * O_STRIDE + 4 * c4) * 4), b = lds128(sO + ((MAXR + r) * O_STRIDE + 4 * c4) * 4);
    float* po = out + (size_t)r * PROW + 2 + 4 * c4;
    *(float2*)po = make_float2(__uint_as_float(a.x) + __uint_as_float(b.x), __uint_as_float(a.y) + __uint_as_float(b.y));
    *(float2*)(po + 2) = make_float2(__uint_as_float(a.z) + __uint_as_float(b.z), __uint_as_float(a.w) + __uint_as_float(b.w));
  }
  if (tid < R) {
    const int r = tid;
    const float m0 = ldsf(sbase + OFF_M1 + r * 4), m1 = ldsf(sbase + OFF_M1 + (MAXR + r) * 4);
    const float M = fmaxf(m0, m1);
    const float f0 = ex2((m0 - M) * LOG2E), f1 = ex2((m1 - M) * LOG2E);
    float l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
      l0 += ldsf(sbase + OFF_L + (w * MAXR + r) * 4);
      l1 += ldsf(sbase + OFF_L + ((4 + w) * MAXR + r) * 4);
    }
    float* po = out + (size_t)r * PROW;
    po[0] = M;
    po[1] = l0 * f0 + l1 * f1;
  }
  if (tid == 0) stamp(7);
  if (has_pool && tid == 0) {
    // Both issuing lanes of this CTA have drawn their last pool tile. The last CTA of the grid to say so
    // puts the counters back to zero for the next launch.
    __threadfence();
    const int total = gridDim.x * gridDim.y;
    if (atomicAdd(p.sched + 32, 1) == total - 1) {
      for (int k = 0; k < (int)gridDim.y; k++) p.sched[k] = 0;
      p.sched[32] = 0;
      __threadfence();
    }
  }
  drain_after_abort(abort_flag);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int NT>
int launch_wt_nt(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                 const DecodeParams& p, bool paged, int nseq, cudaStream_t s) {
  const dim3 grid(p.nch, p.nkvh, nseq);
  if (paged)
    Q27B_CK(launch_pdl(decode_wt_kernel<NT, true>, grid, dim3(WT_THREADS), WT_SMEM_BYTES, s, *kv, *ks, *vv, *vs, p));
  else
    Q27B_CK(launch_pdl(decode_wt_kernel<NT, false>, grid, dim3(WT_THREADS), WT_SMEM_BYTES, s, *kv, *ks, *vv, *vs, p));
  return Q27B_OK;
}

}  // namespace

int launch_decode_wt(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                     const DecodeParams& p, bool paged, int nseq, cudaStream_t s) {
  static bool attr[64] = {};
  static std::mutex attr_mu;
  int dev;
  Q27B_CK(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(attr_mu);
    if (!attr[dev]) {
      Q27B_CK(cudaFuncSetAttribute(decode_wt_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WT_SMEM_BYTES));
      Q27B_CK(cudaFuncSetAttribute(decode_wt_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WT_SMEM_BYTES));
      Q27B_CK(cudaFuncSetAttribute(decode_wt_kernel<3, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, WT_SMEM_BYTES));
      Q27B_CK(cudaFuncSetAttribute(decode_wt_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WT_SMEM_BYTES));
      Q27B_CK(cudaFuncSetAttribute(decode_wt_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WT_SMEM_BYTES));
      Q27B_CK(cudaFuncSetAttribute(decode_wt_kernel<3, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, WT_SMEM_BYTES));
      attr[dev] = true;
    }
  }
  const int nt = (GQA * p.T + 7) / 8;
  if (nt == 1) return launch_wt_nt<1>(kv, ks, vv, vs, p, paged, nseq, s);
  if (nt == 2) return launch_wt_nt<2>(kv, ks, vv, vs, p, paged, nseq, s);
  return launch_wt_nt<3>(kv, ks, vv, vs, p, paged, nseq, s);
}

}  // namespace q27b
