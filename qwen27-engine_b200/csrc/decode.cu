// Split-K flash-decode over a q8_0 or f16 KV cache for 1..4 speculative-verify query tokens.
//
// Replaces attn_mma_kernel + the host wrapper attn_decode of the reference (src/attn.cu:95-292,
// 894-918). Same decomposition of the work (one CTA per (position chunk, KV head), all 6*T query
// rows of the KV head in the CTA, so each K/V byte leaves HBM once; per-chunk partials (m, l, O)
// merged by the log-sum-exp kernel) and the same roundings (Q*scale -> f16, K/V -> f16(int8 * f16
// scale), P -> f16, f32 accumulation, row sums from the f32 P; src/attn.cu:10-11). The kernel
// itself is built for B200:
//
//  * 64-position tiles (K and V values as 128-byte-swizzled 64x128 B boxes, plus for q8_0 the two
//    64x16 B scale boxes) are streamed by TMA into an mbarrier ring (6 stages of 34 KB for q8_0,
//    3 of 64 KB for f16). A stage is refilled by one elected lane right after the group barrier
//    that proves all four warps are done with it, so there is no producer warp and no "empty"
//    barrier: ~140 KB stay in flight per SM, which is what HBM3e needs to stay busy.
//  * Eight consumer warps in two groups of four; the groups take alternate tiles and keep their
//    own running (m, l, O), merged once at the end. Within a group, warp w computes
//    S^T = K Q^T for tile rows 16w..16w+15 (positions on the MMA M axis, the 6*T query rows on
//    N = 8/16/24: no padding waste), then O^T += V^T P^T for head dims 64w..64w+63 over all 64
//    positions. P (64 x 24 f16) is the only thing exchanged between warps.
//  * K and V go from shared memory straight into mma.sync fragments: each lane loads 16 (K) or
//    8 (V) consecutive bytes of a row, and for q8_0 the byte -> f16 conversion (0x64xx magic,
//    minus 1152, times the block scale: one rounding) happens in registers. The contraction index
//    of an MMA may be permuted freely, so the k-slots are chosen to match what a coalesced 16-byte
//    load delivers; Q is pre-permuted to match, once, into registers. With the 128-byte swizzle
//    and a bit-reversed row order inside each 16-row slab every shared-memory load is
//    conflict-free.
//  * The reference maxima of a group only move when a score exceeds them by more than TAU (and on
//    the group's first tile): a tile normally costs one group barrier and no rescale of O.
#define Q27B_INLINE_WAITS  // all eight warps of this kernel run the same code: the wait loops stay inline
#include "combine.h"
#include "common.cuh"
#include "decode_params.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <mutex>

namespace q27b {
namespace {

constexpr int TILE = 64;                       // positions per tile
#ifndef Q27B_NSTAGE
#define Q27B_NSTAGE 6
#endif
#ifndef Q27B_NGROUP
#define Q27B_NGROUP 2
#endif
constexpr int NGROUP = Q27B_NGROUP;            // groups of four warps; group g takes tiles g, g + NGROUP, ...

// Geometry of one pipeline stage. Values: ROWB bytes per position = NSEG segments of 128 bytes, each
// segment stored as a [64 rows][128 B] swizzled box; q8_0 adds [64][16 B] scale boxes.
template <bool Q8>
struct Geo {
  static constexpr int ROWB = Q8 ? AD : 2 * AD;
  static constexpr int NSEG = ROWB / 128;
  static constexpr int SEG_BYTES = TILE * 128;
  static constexpr int VAL_BYTES = NSEG * SEG_BYTES;
  static constexpr int SC_BYTES = Q8 ? TILE * 16 : 0;
  static constexpr int STAGE_BYTES = 2 * VAL_BYTES + 2 * SC_BYTES;  // 34816 (q8_0) / 65536 (f16)
  static constexpr int NSTAGE = Q8 ? Q27B_NSTAGE : 3;
  static constexpr int OFF_KV = 0, OFF_VV = VAL_BYTES, OFF_KS = 2 * VAL_BYTES, OFF_VS = 2 * VAL_BYTES + SC_BYTES;
};
constexpr int RING_BYTES = Geo<true>::NSTAGE * Geo<true>::STAGE_BYTES > Geo<false>::NSTAGE * Geo<false>::STAGE_BYTES
                               ? Geo<true>::NSTAGE * Geo<true>::STAGE_BYTES
                               : Geo<false>::NSTAGE * Geo<false>::STAGE_BYTES;
constexpr int MAX_STAGES = Geo<true>::NSTAGE > Geo<false>::NSTAGE ? Geo<true>::NSTAGE : Geo<false>::NSTAGE;
constexpr int P_STRIDE = 36;                   // words per P row (32 position pairs + 4 padding: no bank conflicts)
constexpr int P_WORDS = MAXR * P_STRIDE;
constexpr int OFF_P = RING_BYTES;                           // [groups][2 buffers][24][36] words
constexpr int OFF_MAX = OFF_P + NGROUP * 2 * P_WORDS * 4;   // [groups][2 buffers][4 warps][24] floats
constexpr int OFF_L = OFF_MAX + NGROUP * 2 * 4 * MAXR * 4;  // [groups][4 warps][24] floats
constexpr int OFF_M1 = OFF_L + NGROUP * 4 * MAXR * 4;       // [groups][24] floats: reference maxima at the end
constexpr int OFF_BAR = OFF_M1 + NGROUP * MAXR * 4;         // full[stages]
constexpr int OFF_FLAG = OFF_BAR + MAX_STAGES * 8;
constexpr int OFF_TOK = OFF_FLAG + 16;                      // [groups][2 buffers] words: "move the maxima" tokens
constexpr int SMEM_USED = OFF_TOK + 32;
constexpr float TAU = 8.0f;                                 // a score may exceed the reference max by this much
constexpr int SMEM_BYTES = SMEM_USED + 1024;               // slack for the 1024-byte alignment of the ring
constexpr int O_STRIDE = AD + 4;                            // floats per row of the end-of-kernel O exchange
static_assert((NGROUP - 1) * MAXR * O_STRIDE * 4 <= RING_BYTES, "O exchange must fit in the ring");
static_assert(NGROUP == 2, "the register budget (Q fragments in registers) is sized for two groups");
static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");

constexpr int N_THREADS = NGROUP * 128;
constexpr int BAR_ALL = 1 + NGROUP;                         // named barrier of all threads (1 .. NGROUP: the groups)

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
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v)); }
__device__ __forceinline__ void stsf(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v)); }
__device__ __forceinline__ float ldsf(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ void bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) { return __byte_perm(a, b, sel); }

// Row of a 16-row slab that MMA row slot s (0..15) stands for: 8 * (s >> 3) + bitrev3(s & 7).
__device__ __forceinline__ int slot_row(int s) { return (s & 8) | ((s & 1) << 2) | (s & 2) | ((s & 4) >> 2); }

// First of the 4 head dims that k-step ks (0..15) of the S^T MMAs covers for lane quarter tg.
// q8_0: a 16-byte load is 16 dims = 4 k-steps; f16: a 16-byte load is 8 dims = 2 k-steps.
template <bool Q8>
__device__ __forceinline__ int ks_dim0(int ks, int tg) {
  if (Q8) return 128 * (ks >> 3) + 64 * ((ks >> 2) & 1) + 16 * tg + 4 * (ks & 3);
  return 64 * (ks >> 2) + 32 * ((ks >> 1) & 1) + 8 * tg + 4 * (ks & 1);
}

// NT = 8-row groups of query rows (ceil(6 T / 8)). PAGED: batched decode over 256-position pages
// (q8_0 only). Q8: q8_0 cache (else f16).
template <int NT, bool PAGED, bool Q8>
__global__ void __launch_bounds__(N_THREADS, 1)
decode_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_ks,
              const __grid_constant__ CUtensorMap tm_vv, const __grid_constant__ CUtensorMap tm_vs,
              const DecodeParams p) {
  using G = Geo<Q8>;
  constexpr int NSTAGE = G::NSTAGE;
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  uint64_t* full = (uint64_t*)(sgen + OFF_BAR);
  volatile int* abort_flag = (volatile int*)(sgen + OFF_FLAG);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {  // start fetching the tensor maps while the position is being read
    tma_prefetch_desc(&tm_kv);
    tma_prefetch_desc(&tm_vv);
    if (Q8) {
      tma_prefetch_desc(&tm_ks);
      tma_prefetch_desc(&tm_vs);
    }
  }
  const int ch = blockIdx.x, kh = blockIdx.y;
  const int T = p.T, R = GQA * T;
  const int seq = PAGED ? blockIdx.z : 0;
  const int pos0 = PAGED ? p.seq_len[seq] - T : *p.pos0;
  const float* qn = p.qn + (size_t)seq * T * p.nqh * AD;
  const int g = lane >> 2, tg = lane & 3;

  // Local rows to attend, and this CTA's chunk [c0, c1) of them (multiples of TILE).
  int n = pos0 + T - p.base_pos;
  if (p.n_local >= 0) n = min(n, p.n_local);
  n = max(0, min(n, p.n_ctx));
  int chunk;
  if (PAGED) {
    chunk = p.chunk_len;
  } else {
    chunk = (n + p.nch - 1) / p.nch;
    chunk = max(TILE, (chunk + TILE - 1) / TILE * TILE);
  }
  const int c0 = min(n, ch * chunk), c1 = min(n, c0 + chunk);
  float* out = p.part + (((size_t)seq * p.nkvh + kh) * p.nch + ch) * MAXR * PROW;

  if (c0 >= c1) {
    // Empty chunk: neutral partial (src/attn.cu:117-120). The paged merge reads only the chunks
    // that a sequence has, so there nothing is written.
    if (!PAGED)
      for (int i = tid; i < R * PROW; i += N_THREADS) out[i] = (i % PROW == 0) ? M_INIT : 0.f;
    return;
  }
  const int ntiles = (c1 - c0 + TILE - 1) / TILE;

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; s++) mbar_init(&full[s], 1);
    *abort_flag = 0;
    for (int i = 0; i < 2 * NGROUP; i++) ((volatile uint32_t*)(sgen + OFF_TOK))[i] = 0;
    mbar_fence_init();
  }
  __syncthreads();

  // TMA of tile `it` into stage it % NSTAGE (one thread).
  const int row0 = kh * p.n_ctx + c0;
  auto issue_tile = [&](int it) {
    const int s = it % NSTAGE;
    uint8_t* st = sgen + (size_t)s * G::STAGE_BYTES;
    mbar_expect_tx(&full[s], G::STAGE_BYTES);
    int row = row0 + it * TILE;
    if (PAGED) {  // a tile never straddles a page (64 | 256)
      const int pp = c0 + it * TILE;
      int pg = p.page_table[(size_t)seq * p.max_pages + pp / Q27B_PAGE];
      if (pg < 0 || pg >= p.n_pages) {  // never read outside the pool: flag it and read page 0
        atomicOr(p.status, ST_BAD_PAGE);
        pg = 0;
      }
      row = (pg * p.nkvh + kh) * Q27B_PAGE + pp % Q27B_PAGE;
    }
#pragma unroll
    for (int sg = 0; sg < G::NSEG; sg++) {
      tma_load_2d(st + G::OFF_KV + sg * G::SEG_BYTES, &tm_kv, 128 * sg, row, &full[s]);
      tma_load_2d(st + G::OFF_VV + sg * G::SEG_BYTES, &tm_vv, 128 * sg, row, &full[s]);
    }
    if (Q8) {
      tma_load_2d(st + G::OFF_KS, &tm_ks, 0, row, &full[s]);
      tma_load_2d(st + G::OFF_VS, &tm_vs, 0, row, &full[s]);
    }
  };

  const int grp = warp >> 2, wq = warp & 3;
  const bool loader = wq == 0 && lane == 0;  // refills this group's stages
  if (loader)
    for (int it = grp; it < min(ntiles, NSTAGE); it += NGROUP) issue_tile(it);
  const int ra = 16 * wq + slot_row(g), rb = ra + 8;  // tile rows of MMA row slots g and g + 8 (S^T)

  // Q fragments (B operand of S^T = K Q^T), permuted to the k-slot order of the K loads:
  // k-step ks covers dims ks_dim0(ks, tg) .. +3 of query row 8nt + g.
  uint32_t qf[16][NT][2];
#pragma unroll
  for (int ks = 0; ks < 16; ks++) {
    const int dim0 = ks_dim0<Q8>(ks, tg);
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      const int r = 8 * nt + g;
      uint32_t b0 = 0, b1 = 0;
      if (r < R) {
        const float4 q = *(const float4*)(qn + ((size_t)(r / GQA) * p.nqh + kh * GQA + r % GQA) * AD + dim0);
        b0 = pack_h2(q.x * p.kq_scale, q.y * p.kq_scale);
        b1 = pack_h2(q.z * p.kq_scale, q.w * p.kq_scale);
      }
      qf[ks][nt][0] = b0;
      qf[ks][nt][1] = b1;
    }
  }



  // Visible end (local row index, exclusive) of this lane's query rows 8nt + 2tg + e.
  int lim[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int e = 0; e < 2; e++) {
      const int r = 8 * nt + 2 * tg + e;
      lim[nt][e] = min(c1, pos0 + min(r / GQA, T - 1) + 1 - p.base_pos);
    }
  const int lim_min = min(c1, pos0 + 1 - p.base_pos);

  float o[4][NT][4];
#pragma unroll
  for (int mt = 0; mt < 4; mt++)
#pragma unroll
    for (int nt = 0; nt < NT; nt++) o[mt][nt][0] = o[mt][nt][1] = o[mt][nt][2] = o[mt][nt][3] = 0.f;
  float m[NT][2], l[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    m[nt][0] = m[nt][1] = M_INIT;
    l[nt][0] = l[nt][1] = 0.f;
  }

  const uint32_t sP = sbase + OFF_P + grp * 2 * P_WORDS * 4;
  const uint32_t sMax = sbase + OFF_MAX + grp * 2 * 4 * MAXR * 4;
  const uint32_t sTok = sbase + OFF_TOK + grp * 8;
  const uint32_t sel_sc = (tg & 2) ? 0x3232u : 0x1010u;  // which f16 of a scale word this lane's K blocks use
  const uint32_t MAGIC = 0x64646464u;
  // Byte offsets inside a stage that do not depend on the tile (q8_0 layout). K: chunk tg of rows
  // ra / rb in a segment; chunk 4 + tg is the same address with bit 6 flipped. V: 8 bytes of rows
  // slot_row(tg) (+8) and slot_row(tg) + 1 (+8) in this warp's 64-dim quarter; 16 positions further
  // is 2048 bytes further. Scales: this lane's block of those rows.
  const uint32_t kA = G::OFF_KV + ra * 128 + ((tg ^ (ra & 7)) << 4);
  const uint32_t kB = G::OFF_KV + rb * 128 + ((tg ^ (rb & 7)) << 4);
  const uint32_t vrow = slot_row(tg), vcb = (wq & 1) * 4 + (g >> 1);
  const uint32_t vQ = G::OFF_VV + (wq >> 1) * G::SEG_BYTES + (g & 1) * 8;
  const uint32_t vA = vQ + vrow * 128 + ((vcb ^ (vrow & 7)) << 4);
  const uint32_t vC = vQ + (vrow + 1) * 128 + ((vcb ^ ((vrow + 1) & 7)) << 4);
  const uint32_t sA = G::OFF_VS + (2 * wq + (g >> 2)) * 2 + vrow * 16;

  int jt = 0;
  for (int it = grp; it < ntiles; it += NGROUP, jt++) {
    const int s = it % NSTAGE;
    mbar_wait(&full[s], (it / NSTAGE) & 1, abort_flag, p.status);
    const uint32_t st = sbase + s * G::STAGE_BYTES;
    const int tile_p0 = c0 + it * TILE;
    const bool edge = tile_p0 + TILE > lim_min;  // some row of the tile is masked for some query row

    // ---- S^T = K Q^T for tile rows ra, rb
    // (two accumulator sets, alternating, so that consecutive MMAs do not depend on each other)
    float sacc[NT][4], sacc2[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
      sacc2[nt][0] = sacc2[nt][1] = sacc2[nt][2] = sacc2[nt][3] = 0.f;
    }
    if constexpr (Q8) {
      const uint4 sca = lds128(st + G::OFF_KS + ra * 16), scb = lds128(st + G::OFF_KS + rb * 16);
      const uint32_t scaw[4] = {sca.x, sca.y, sca.z, sca.w}, scbw[4] = {scb.x, scb.y, scb.z, scb.w};
#pragma unroll
      for (int hj = 0; hj < 4; hj++) {
        const int h = hj >> 1, j = hj & 1;
        const uint4 xa = lds128(st + (kA ^ (j << 6)) + h * G::SEG_BYTES);  // = swz128(ra, 4j + tg)
        const uint4 xb = lds128(st + (kB ^ (j << 6)) + h * G::SEG_BYTES);
        const __half2 da = u32_as_h2(prmt(scaw[hj], scaw[hj], sel_sc));
        const __half2 db = u32_as_h2(prmt(scbw[hj], scbw[hj], sel_sc));
        const uint32_t xaw[4] = {xa.x, xa.y, xa.z, xa.w}, xbw[4] = {xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int s2 = 0; s2 < 4; s2++) {
          const uint32_t wa = xaw[s2] ^ 0x80808080u, wb = xbw[s2] ^ 0x80808080u;
          const uint32_t a0 = dq_pair(prmt(wa, MAGIC, 0x4140), da), a2 = dq_pair(prmt(wa, MAGIC, 0x4342), da);
          const uint32_t a1 = dq_pair(prmt(wb, MAGIC, 0x4140), db), a3 = dq_pair(prmt(wb, MAGIC, 0x4342), db);
          const int ks = 4 * hj + s2;
#pragma unroll
          for (int nt = 0; nt < NT; nt++)
            mma16816((hj & 1) ? sacc2[nt] : sacc[nt], a0, a1, a2, a3, qf[ks][nt][0], qf[ks][nt][1]);
        }
      }
    } else {
#pragma unroll
      for (int sj = 0; sj < 8; sj++) {  // segment sj >> 1 (64 dims), 16-byte chunk 4 (sj & 1) + tg of it
        const uint4 xa = lds128(st + G::OFF_KV + (sj >> 1) * G::SEG_BYTES + swz128(ra, 4 * (sj & 1) + tg));
        const uint4 xb = lds128(st + G::OFF_KV + (sj >> 1) * G::SEG_BYTES + swz128(rb, 4 * (sj & 1) + tg));
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          mma16816(sacc[nt], xa.x, xb.x, xa.y, xb.y, qf[2 * sj][nt][0], qf[2 * sj][nt][1]);
          mma16816(sacc2[nt], xa.z, xb.z, xa.w, xb.w, qf[2 * sj + 1][nt][0], qf[2 * sj + 1][nt][1]);
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
    // its tile maxima, m, l and O are rescaled and P is recomputed. Otherwise - almost always - a
    // tile costs one group barrier and no rescale; P stays <= e^TAU, well inside f16.
    const int buf = jt & 1;
    const uint32_t token = (uint32_t)(jt + 1);
    bool exceed = jt == 0;
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) exceed |= fmaxf(sacc[nt][e], sacc[nt][2 + e]) > m[nt][e] + TAU;
    if (__any_sync(0xffffffffu, exceed) && lane == 0) sts32(sTok + buf * 4, token);
    float lt[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const float mb = m[nt][e] * LOG2E;
        const float pa = ex2(fmaf(sacc[nt][e], LOG2E, -mb)), pb = ex2(fmaf(sacc[nt][2 + e], LOG2E, -mb));
        lt[nt][e] = pa + pb;
        // position pair (slot g, slot g + 8) of warp wq = P^T k-slot pair 8wq + g
        sts32(sP + (buf * P_WORDS + (8 * nt + 2 * tg + e) * P_STRIDE + 8 * wq + g) * 4, pack_h2(pa, pb));
      }
    bar_sync(1 + grp, 128);
    // All four warps are past the previous tile of this group: its stage can be refilled.
    if (loader && jt >= 1 && it - NGROUP + NSTAGE < ntiles) issue_tile(it - NGROUP + NSTAGE);
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
      bar_sync(1 + grp, 128);
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
#pragma unroll
          for (int mt = 0; mt < 4; mt++) {
            o[mt][nt][e] *= f;
            o[mt][nt][2 + e] *= f;
          }
          const float mb = mn * LOG2E;
          const float pa = ex2(fmaf(sacc[nt][e], LOG2E, -mb)), pb = ex2(fmaf(sacc[nt][2 + e], LOG2E, -mb));
          lt[nt][e] = pa + pb;
          sts32(sP + (buf * P_WORDS + r * P_STRIDE + 8 * wq + g) * 4, pack_h2(pa, pb));
        }
      bar_sync(1 + grp, 128);
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
      l[nt][0] += lt[nt][0];
      l[nt][1] += lt[nt][1];
    }

    // ---- O^T += V^T P^T for head dims 64wq + 8g .. +7 (8 values of each V row per lane)
    {
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
        if constexpr (Q8) {
          // rows pa, pb = pa + 8 share one swizzle term, pc = pa + 1, pd = pa + 9 the other
          const uint2 xa = lds64(st + vA + ks * 2048), xb = lds64(st + vA + ks * 2048 + 1024);
          const uint2 xc = lds64(st + vC + ks * 2048), xd = lds64(st + vC + ks * 2048 + 1024);
          uint32_t sa = ldsu16(st + sA + ks * 256), sb = ldsu16(st + sA + ks * 256 + 128);
          uint32_t scc = ldsu16(st + sA + ks * 256 + 16), sd = ldsu16(st + sA + ks * 256 + 144);
          if (edge) {  // rows past the end of the sequence may hold anything: make them exact zeros
            if (tile_p0 + pa >= c1) sa = 0;
            if (tile_p0 + pb >= c1) sb = 0;
            if (tile_p0 + pc >= c1) scc = 0;
            if (tile_p0 + pd >= c1) sd = 0;
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
        } else {
          // f16: segment wq holds dims 64wq .. 64wq+63; chunk g of a row = dims 64wq + 8g .. +7
          const uint32_t vbase = st + G::OFF_VV + wq * G::SEG_BYTES;
          uint4 xa = lds128(vbase + swz128(pa, g)), xb = lds128(vbase + swz128(pb, g));
          uint4 xc = lds128(vbase + swz128(pc, g)), xd = lds128(vbase + swz128(pd, g));
          if (edge) {  // rows past the end of the sequence may hold anything: make them exact zeros
            if (tile_p0 + pa >= c1) xa = make_uint4(0, 0, 0, 0);
            if (tile_p0 + pb >= c1) xb = make_uint4(0, 0, 0, 0);
            if (tile_p0 + pc >= c1) xc = make_uint4(0, 0, 0, 0);
            if (tile_p0 + pd >= c1) xd = make_uint4(0, 0, 0, 0);
          }
          const uint32_t xaw[4] = {xa.x, xa.y, xa.z, xa.w}, xbw[4] = {xb.x, xb.y, xb.z, xb.w};
          const uint32_t xcw[4] = {xc.x, xc.y, xc.z, xc.w}, xdw[4] = {xd.x, xd.y, xd.z, xd.w};
#pragma unroll
          for (int mt = 0; mt < 4; mt++) {
            // word mt of a row = dims 2mt (d-slot g) and 2mt+1 (d-slot g+8); pair them across positions
            const uint32_t a0 = prmt(xaw[mt], xbw[mt], 0x5410), a1 = prmt(xaw[mt], xbw[mt], 0x7632);
            const uint32_t a2 = prmt(xcw[mt], xdw[mt], 0x5410), a3 = prmt(xcw[mt], xdw[mt], 0x7632);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) mma16816(o[mt][nt], a0, a1, a2, a3, b0[nt], b1[nt]);
          }
        }
      }
    }
  }

  // ---- row sums over this warp's positions
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int e = 0; e < 2; e++) {
      float v = l[nt][e];
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      l[nt][e] = v;
      if (g == 0) stsf(sbase + OFF_L + ((grp * 4 + wq) * MAXR + 8 * nt + 2 * tg + e) * 4, v);
    }
  if (wq == 0 && g == 0) {
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) stsf(sbase + OFF_M1 + (grp * MAXR + 8 * nt + 2 * tg + e) * 4, m[nt][e]);
  }
  bar_sync(BAR_ALL, N_THREADS);  // every tile consumed: the ring is free for the O exchange

  // ---- merge the groups (log-sum-exp) and write the chunk partial
  const uint32_t sO = sbase;
  if (grp > 0) {
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int r = 8 * nt + 2 * tg + e;
#pragma unroll
        for (int mt = 0; mt < 4; mt++) {
          const int d = 64 * wq + 8 * g + 2 * mt;
          stsf(sO + (((grp - 1) * MAXR + r) * O_STRIDE + d) * 4, o[mt][nt][e]);
          stsf(sO + (((grp - 1) * MAXR + r) * O_STRIDE + d + 1) * 4, o[mt][nt][2 + e]);
        }
      }
  }
  bar_sync(BAR_ALL, N_THREADS);
  if (grp == 0) {
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const int r = 8 * nt + 2 * tg + e;
        if (r >= R) continue;
        float mg[NGROUP], f[NGROUP];
        float M = m[nt][e];
#pragma unroll
        for (int k = 1; k < NGROUP; k++) {
          mg[k] = ldsf(sbase + OFF_M1 + (k * MAXR + r) * 4);
          M = fmaxf(M, mg[k]);
        }
        f[0] = ex2((m[nt][e] - M) * LOG2E);
#pragma unroll
        for (int k = 1; k < NGROUP; k++) f[k] = ex2((mg[k] - M) * LOG2E);
        float* po = out + (size_t)r * PROW;
#pragma unroll
        for (int mt = 0; mt < 4; mt++) {
          const int d = 64 * wq + 8 * g + 2 * mt;
          float v0 = o[mt][nt][e] * f[0], v1 = o[mt][nt][2 + e] * f[0];
#pragma unroll
          for (int k = 1; k < NGROUP; k++) {
            v0 += ldsf(sO + (((k - 1) * MAXR + r) * O_STRIDE + d) * 4) * f[k];
            v1 += ldsf(sO + (((k - 1) * MAXR + r) * O_STRIDE + d + 1) * 4) * f[k];
          }
          *(float2*)(po + 2 + d) = make_float2(v0, v1);
        }
        if (wq == 0 && g == 0) {
          float lsum = 0.f;
#pragma unroll
          for (int k = 0; k < NGROUP; k++) {
            float lk = 0.f;
#pragma unroll
            for (int w = 0; w < 4; w++) lk += ldsf(sbase + OFF_L + ((k * 4 + w) * MAXR + r) * 4);
            lsum += lk * f[k];
          }
          po[0] = M;
          po[1] = lsum;
        }
      }
  }
}

// Tensor maps of one cache (values and, for q8_0, scales), by value, from the process-wide cache.
int get_tmaps(const void* cache, int nkvh, int n_ctx, bool q8, CUtensorMap* vals, CUtensorMap* scales) {
  const uint64_t rows = (uint64_t)nkvh * n_ctx;
  if (q8) return q8_tmaps(cache, rows, vals, scales);
  if (int rc = cached_tmap_2d(vals, cache, rows, 2 * AD, 2 * AD, 128, TILE, true)) return rc;
  *scales = *vals;  // unused by the f16 kernel
  return Q27B_OK;
}

// Per-device one-time set-up flags of this file's kernels (attribute opt-ins), safe from several threads.
std::mutex g_setup_mu;

template <int NT, bool PAGED, bool Q8>
int launch_decode(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                  const DecodeParams& p, int nseq, cudaStream_t s) {
  static bool attr[64] = {};
  int dev;
  Q27B_CK(cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (!attr[dev]) {
      Q27B_CK(cudaFuncSetAttribute(decode_kernel<NT, PAGED, Q8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
      attr[dev] = true;
    }
  }
  Q27B_CK(launch_pdl(decode_kernel<NT, PAGED, Q8>, dim3(p.nch, p.nkvh, nseq), dim3(N_THREADS), SMEM_BYTES, s, *kv, *ks, *vv,
                     *vs, p));
  return Q27B_OK;
}
template <bool PAGED, bool Q8>
int launch_decode_t(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                    const DecodeParams& p, int nseq, cudaStream_t s) {
  const int nt = (GQA * p.T + 7) / 8;
  if (nt == 1) return launch_decode<1, PAGED, Q8>(kv, ks, vv, vs, p, nseq, s);
  if (nt == 2) return launch_decode<2, PAGED, Q8>(kv, ks, vv, vs, p, nseq, s);
  return launch_decode<3, PAGED, Q8>(kv, ks, vv, vs, p, nseq, s);
}

// Which split-K kernel serves a q8_0 cache: the warp-specialised kernel of decode_ws.cu unless
// Q27B_DECODE_KERNEL=mma|tc|wt or q27b_set_decode_kernel(1|2|4) asks for the single-role warp-MMA kernel of
// this file, the tcgen05 kernel (decode_tc.cu) or the warp-specialised kernel with P V on tcgen05 (decode_wt.cu). Measured on B200 (same call, 20 calls in a CUDA
// graph, 150k positions, T = 4): warp-specialised 69.7 us per call, single-role 75.7 us, tcgen05
// 73.7-80.8 us depending on the build (eight differently specialised warp roles with a serial hand-off
// chain: sensitive to code layout). f16 caches always use the kernel of this file.
// Whether the CTAs of the warp-specialised kernel share a pool of tiles (see decode_ws.cu) or keep to
// equal static shares (Q27B_DECODE_POOL=0, q27b_set_decode_schedule(0)): the static form gives the
// same bits on every run, the pool form ends earlier.
std::atomic<bool> g_pool_schedule{[] {
  const char* e = getenv("Q27B_DECODE_POOL");
  return !(e && e[0] == '0');
}()};
std::atomic<int> g_kernel_choice{-1};  // -1: not read yet; 0 default (= 3), 1 single-role warp-MMA, 2 tcgen05, 3 warp-specialised, 4 the same with P V on tcgen05
int kernel_choice() {
  int k = g_kernel_choice.load(std::memory_order_relaxed);
  if (k < 0) {
    const char* e = getenv("Q27B_DECODE_KERNEL");
    k = !e ? 0 : e[0] == 'm' ? 1 : e[0] == 't' ? 2 : (e[0] == 'w' && e[1] == 't') ? 4 : e[0] == 'w' ? 3 : 0;
    int expected = -1;
    if (!g_kernel_choice.compare_exchange_strong(expected, k)) k = expected;
  }
  return k;
}
// Launches the split-K kernel chosen for a q8_0 cache.
int launch_q8(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
              const DecodeParams& p, bool paged, int nseq, cudaStream_t s, bool single_group = false) {
  const int k = kernel_choice();
  if (k == 2) return launch_decode_tc(kv, ks, vv, vs, p, paged, nseq, s);
  if (k == 0 || k == 3) return launch_decode_ws(kv, ks, vv, vs, p, paged, nseq, s, single_group);
  if (k == 4) return launch_decode_wt(kv, ks, vv, vs, p, paged, nseq, s);
  return paged ? launch_decode_t<true, true>(kv, ks, vv, vs, p, nseq, s) : launch_decode_t<false, true>(kv, ks, vv, vs, p, nseq, s);
}

// Records a measurement event on s; in a stream that is being captured the record becomes an event
// node of the graph (cudaEventRecordExternal), so that it is taken again at every replay.
int record_hook(cudaEvent_t ev, cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  Q27B_CK(cudaStreamIsCapturing(s, &st));
  Q27B_CK(cudaEventRecordWithFlags(ev, s, st == cudaStreamCaptureStatusActive ? cudaEventRecordExternal : cudaEventRecordDefault));
  return Q27B_OK;
}

// Split-K pass of one sequence into the decode workspace [nkvh][nch][24][258].
int decode_split(DeviceCtx* ctx, const float* qn, const void* kcache, const void* vcache, const int* pos0, int T,
                 float kq_scale, int nqh, int nkvh, int n_ctx, int q8, int base_pos, int n_local, int* nch_out,
                 cudaStream_t s) {
  if (nkvh > ctx->n_sm) return fail(Q27B_BAD_SHAPE, "attn_decode: more KV heads than SMs");
  const int nch = std::max(1, ctx->n_sm / nkvh);
  float* part;
  if (int rc = decode_ws(ctx, &part)) return rc;
  CUtensorMap kvm, ksm, vvm, vsm;
  if (int rc = get_tmaps(kcache, nkvh, n_ctx, q8 != 0, &kvm, &ksm)) return rc;
  if (int rc = get_tmaps(vcache, nkvh, n_ctx, q8 != 0, &vvm, &vsm)) return rc;
  const CUtensorMap *kv = &kvm, *ks = &ksm, *vv = &vvm, *vs = &vsm;
  DecodeParams p = {};
  p.qn = qn; p.part = part; p.pos0 = pos0; p.status = ctx->status;
  p.T = T; p.nqh = nqh; p.nkvh = nkvh; p.n_ctx = n_ctx; p.nch = nch; p.kq_scale = kq_scale;
  p.base_pos = base_pos; p.n_local = n_local; p.trace = ctx->trace;
  p.sched = (g_pool_schedule.load(std::memory_order_relaxed) && nkvh <= 32) ? ctx->status + 16 : nullptr;
  *nch_out = nch;
  if (ctx->split_begin)
    if (int rc = record_hook(ctx->split_begin, s)) return rc;
  if (int rc = !q8 ? launch_decode_t<false, false>(kv, ks, vv, vs, p, 1, s) : launch_q8(kv, ks, vv, vs, p, false, 1, s))
    return rc;
  if (ctx->split_event)
    if (int rc = record_hook(ctx->split_event, s)) return rc;
  return Q27B_OK;
}

// ---------------------------------------------------------------- decode without any allocation
// Scratch of q27b_attn_decode_noalloc: the split partials [chunk slots][24 rows][258 floats] and a
// status word (followed, from int 16 on, by the tile counters of the pool schedule, which every launch
// leaves at zero), reserved in the library image itself. NOALLOC_SLOTS chunk slots = nkvh * chunks per
// KV head, which on a GPU with up to 160 SMs is at most 160 (3.96 MB). Every GPU that loads the
// library carries this array until the process exits.
constexpr int NOALLOC_SLOTS = 160;
static __device__ __align__(256) float g_noalloc_part[(size_t)NOALLOC_SLOTS * MAXR * PROW];
static __device__ __align__(256) int g_noalloc_status[64];

// Device addresses of the two arrays, per device. In host code `g_noalloc_part` is only a
// handle for the runtime, not an address a kernel could use: the address has to be asked for, on
// the device in question, with cudaGetSymbolAddress.
float* g_noalloc_part_ptr[64] = {};
int* g_noalloc_status_ptr[64] = {};

int noalloc_setup(int dev) {
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (g_noalloc_part_ptr[dev]) return Q27B_OK;
  float* part = nullptr;
  int* status = nullptr;
  Q27B_CK(cudaGetSymbolAddress((void**)&part, g_noalloc_part));
  Q27B_CK(cudaGetSymbolAddress((void**)&status, g_noalloc_status));
  // the kernels' shared-memory opt-in, done here so that later calls only launch
  if (int rc = decode_ws_setup()) return rc;
  g_noalloc_status_ptr[dev] = status;
  g_noalloc_part_ptr[dev] = part;
  return Q27B_OK;
}

}  // namespace

// Reads (and clears) the status word that the no-allocation entry point's kernels report into; 0 when
// that entry point has not run on this device. Copies from the library's own device array: allocates nothing.
int noalloc_status(int dev, int* out) {
  *out = 0;
  int* ptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mu);
    ptr = (dev >= 0 && dev < 64) ? g_noalloc_status_ptr[dev] : nullptr;
  }
  if (!ptr) return Q27B_OK;
  Q27B_CK(cudaMemcpy(out, ptr, sizeof(int), cudaMemcpyDeviceToHost));
  if (*out) Q27B_CK(cudaMemset(ptr, 0, sizeof(int)));
  return Q27B_OK;
}
}  // namespace q27b

using namespace q27b;

extern "C" {

int q27b_attn_decode(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o, int8_t* xq,
                     float* xd, const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8,
                     void* stream) {
  if (T < 1 || T > Q27B_MAX_T || nkvh < 1 || nqh != nkvh * GQA || n_ctx < 1)
    return fail(Q27B_BAD_SHAPE, "attn_decode: bad shape");
  if (!qn || !qg || !kcache || !vcache || !pos0 || (!o && !xq) || (xq && !xd))
    return fail(Q27B_BAD_SHAPE, "attn_decode: null pointer");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  int nch;
  if (int rc = decode_split(ctx, qn, kcache, vcache, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8, 0, -1, &nch,
                            (cudaStream_t)stream))
    return rc;
  if (ctx->split_only) return Q27B_OK;
  MergeParams mp = {};
  mp.part = ctx->dec.p; mp.nparts = nch; mp.rows = (int64_t)T * nqh; mp.qg = qg; mp.o = o; mp.xq = xq; mp.xd = xd;
  mp.T = T; mp.nqh = nqh;
  return launch_merge(mp, true, (cudaStream_t)stream);
}

int q27b_attn_decode_partial(const float* qn, const void* kcache, const void* vcache, float* part, const int* pos0,
                             int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, int base_pos, int n_local,
                             void* stream) {
  if (T < 1 || T > Q27B_MAX_T || nkvh < 1 || nqh != nkvh * GQA || n_ctx < 1 || base_pos < 0 || n_local < 0 ||
      n_local > n_ctx)
    return fail(Q27B_BAD_SHAPE, "attn_decode_partial: bad shape");
  if (!qn || !kcache || !vcache || !pos0 || !part) return fail(Q27B_BAD_SHAPE, "attn_decode_partial: null pointer");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  int nch;
  if (int rc = decode_split(ctx, qn, kcache, vcache, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8, base_pos, n_local, &nch,
                            (cudaStream_t)stream))
    return rc;
  MergeParams mp = {};
  mp.part = ctx->dec.p; mp.nparts = nch; mp.rows = (int64_t)T * nqh; mp.part_out = part; mp.T = T; mp.nqh = nqh;
  return launch_merge(mp, true, (cudaStream_t)stream);
}

int q27b_attn_decode_partial_push(const float* qn, const void* kcache, const void* vcache, const int* pos0, int T,
                                  float kq_scale, int nqh, int nkvh, int n_ctx, int q8, int base_pos, int n_local,
                                  void* const* peer_xbuf, int my_z, int nz, void* stream) {
  if (T < 1 || T > Q27B_MAX_T || nkvh < 1 || nqh != nkvh * GQA || n_ctx < 1 || base_pos < 0 || n_local < 0 ||
      n_local > n_ctx || nz < 1 || nz > 8 || my_z < 0 || my_z >= nz)
    return fail(Q27B_BAD_SHAPE, "attn_decode_partial_push: bad shape");
  if (!qn || !kcache || !vcache || !pos0 || !peer_xbuf) return fail(Q27B_BAD_SHAPE, "attn_decode_partial_push: null pointer");
  for (int k = 0; k < nz; k++)
    if (!peer_xbuf[k]) return fail(Q27B_BAD_SHAPE, "attn_decode_partial_push: null pointer");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  // Every buffer must be device memory that kernels of this GPU may store into: a peer's buffer needs
  // peer access from this device to the peer's, which is enabled here (once per pointer) rather than
  // left to whoever mapped the memory. Anything else is refused before a kernel can touch it.
  for (int k = 0; k < nz; k++)
    if (int rc = check_peer_buffer(peer_xbuf[k], "attn_decode_partial_push")) return rc;
  int nch;
  if (int rc = decode_split(ctx, qn, kcache, vcache, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8, base_pos, n_local, &nch,
                            (cudaStream_t)stream))
    return rc;
  MergeParams mp = {};
  mp.part = ctx->dec.p; mp.nparts = nch; mp.rows = (int64_t)T * nqh; mp.T = T; mp.nqh = nqh;
  for (int k = 0; k < nz; k++) mp.push_buf[k] = peer_xbuf[k];
  mp.push_n = nz; mp.push_z = my_z; mp.xbuf = (int*)peer_xbuf[my_z]; mp.status = ctx->status;
  return launch_merge(mp, true, (cudaStream_t)stream);
}

int q27b_attn_decode_exchange(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                              const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, int base_pos,
                              int n_local, void* const* peer_xbuf, int my_z, int nz, void* stream) {
  if (!o) return fail(Q27B_BAD_SHAPE, "attn_decode_exchange: null pointer");
  if (T < 1 || T > Q27B_MAX_T || nkvh < 1 || nqh != nkvh * GQA || n_ctx < 1 || base_pos < 0 || n_local < 0 ||
      n_local > n_ctx || nz < 1 || nz > 8 || my_z < 0 || my_z >= nz)
    return fail(Q27B_BAD_SHAPE, "attn_decode_exchange: bad shape");
  if (!qn || !kcache || !vcache || !pos0 || !peer_xbuf) return fail(Q27B_BAD_SHAPE, "attn_decode_exchange: null pointer");
  for (int k = 0; k < nz; k++)
    if (!peer_xbuf[k]) return fail(Q27B_BAD_SHAPE, "attn_decode_exchange: null pointer");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  // One kernel after the split-K kernel pushes and merges when a row has many partials and few rows (the shape
  // of a KV-length slice: one or two KV heads on a whole GPU); otherwise the pair of calls does the same.
  const int64_t rows = (int64_t)T * nqh;
  const int nch = std::max(1, ctx->n_sm / nkvh);
  const char* e = getenv("Q27B_MERGE_SLICED");
  // (the CTAs of the fused kernel wait for their peers' CTAs of the same index, so all of them must be resident at
  // once: no more CTAs than SMs)
  const int64_t slices = rows * 4 <= 160 ? 4 : 2;
  const bool fused = nch > 64 && rows * 2 <= 160 && rows * slices <= ctx->n_sm && !(e && e[0] == '0');
  if (!fused) {
    if (int rc = q27b_attn_decode_partial_push(qn, kcache, vcache, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8, base_pos, n_local,
                                               peer_xbuf, my_z, nz, stream))
      return rc;
    return q27b_lse_merge_wait(peer_xbuf[my_z], nz, rows, qg, o, stream);
  }
  for (int k = 0; k < nz; k++)
    if (int rc = check_peer_buffer(peer_xbuf[k], "attn_decode_exchange")) return rc;
  int nch_out;
  if (int rc = decode_split(ctx, qn, kcache, vcache, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8, base_pos, n_local, &nch_out,
                            (cudaStream_t)stream))
    return rc;
  MergeParams mp = {};
  mp.part = ctx->dec.p; mp.nparts = nch_out; mp.rows = rows; mp.T = T; mp.nqh = nqh; mp.qg = qg; mp.o = o;
  for (int k = 0; k < nz; k++) mp.push_buf[k] = peer_xbuf[k];
  mp.push_n = nz; mp.push_z = my_z; mp.xbuf = (int*)peer_xbuf[my_z]; mp.status = ctx->status;
  return launch_merge(mp, true, (cudaStream_t)stream);
}

int q27b_attn_decode_noalloc(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                             int8_t* xq, float* xd, const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx,
                             int q8, void* stream) {
  if (T < 1 || T > Q27B_MAX_T || nkvh < 1 || nqh != nkvh * GQA || n_ctx < 1)
    return fail(Q27B_BAD_SHAPE, "attn_decode_noalloc: bad shape");
  if (!qn || !qg || !kcache || !vcache || !pos0 || (!o && !xq) || (xq && !xd))
    return fail(Q27B_BAD_SHAPE, "attn_decode_noalloc: null pointer");
  if (!q8) return fail(Q27B_UNSUPPORTED, "attn_decode_noalloc: q8_0 KV cache only");
  int dev = 0, n_sm = 0;
  Q27B_CK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(Q27B_UNSUPPORTED, "device index out of range");
  Q27B_CK(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  const int nch = std::max(1, n_sm / nkvh);
  if ((size_t)nkvh * nch > (size_t)NOALLOC_SLOTS)
    return fail(Q27B_BAD_SHAPE, "attn_decode_noalloc: needs " + std::to_string(nkvh * nch) +
                                    " chunk partials, the built-in scratch holds " + std::to_string(NOALLOC_SLOTS) +
                                    " (use q27b_attn_decode, which allocates)");
  if (int rc = noalloc_setup(dev)) return rc;
  CUtensorMap kvm, ksm, vvm, vsm;  // (the tensor-map cache lives in host memory)
  if (int rc = get_tmaps(kcache, nkvh, n_ctx, true, &kvm, &ksm)) return rc;
  if (int rc = get_tmaps(vcache, nkvh, n_ctx, true, &vvm, &vsm)) return rc;
  const CUtensorMap *kv = &kvm, *ks = &ksm, *vv = &vvm, *vs = &vsm;
  DecodeParams p = {};
  p.qn = qn; p.part = g_noalloc_part_ptr[dev]; p.pos0 = pos0; p.status = g_noalloc_status_ptr[dev];
  p.T = T; p.nqh = nqh; p.nkvh = nkvh; p.n_ctx = n_ctx; p.nch = nch; p.kq_scale = kq_scale;
  p.base_pos = 0; p.n_local = -1;
  // the tile counters of the pool schedule sit behind the status word, as in the allocated workspace
  p.sched = (g_pool_schedule.load(std::memory_order_relaxed) && nkvh <= 32) ? g_noalloc_status_ptr[dev] + 16 : nullptr;
  if (int rc = launch_decode_ws(kv, ks, vv, vs, p, false, 1, (cudaStream_t)stream)) return rc;
  MergeParams mp = {};
  mp.part = g_noalloc_part_ptr[dev]; mp.nparts = nch; mp.rows = (int64_t)T * nqh; mp.qg = qg; mp.o = o; mp.xq = xq;
  mp.xd = xd; mp.T = T; mp.nqh = nqh;
  return launch_merge(mp, true, (cudaStream_t)stream);
}

int q27b_set_decode_kernel(int which) {
  if (which < 0 || which > 4)
    return fail(Q27B_BAD_SHAPE, "set_decode_kernel: 0 auto, 1 warp-MMA, 2 tcgen05, 3 warp-specialised, 4 warp-specialised with P V on tcgen05");
  g_kernel_choice.store(which);
  return Q27B_OK;
}

int q27b_set_decode_schedule(int pool) {
  g_pool_schedule.store(pool != 0);
  return Q27B_OK;
}

int q27b_debug_split_event(void* event) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  ctx->split_event = (cudaEvent_t)event;
  ctx->split_begin = nullptr;
  return Q27B_OK;
}

int q27b_debug_split_only(int on) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  ctx->split_only = on != 0;
  return Q27B_OK;
}

int q27b_debug_split_events(void* begin, void* end) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  ctx->split_begin = (cudaEvent_t)begin;
  ctx->split_event = (cudaEvent_t)end;
  return Q27B_OK;
}

int q27b_debug_decode_trace(unsigned long long* stamps) {
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  ctx->trace = stamps;
  return Q27B_OK;
}

int q27b_attn_decode_paged(const float* qn, const float* qg, const void* kpool, const void* vpool,
                           const int* page_table, const int* seq_len, float* o, int B, int T, float kq_scale, int nqh,
                           int nkvh, int n_pages, int max_pages, int max_seq_len, void* stream) {
  if (B < 1 || T < 1 || T > Q27B_MAX_T || nkvh < 1 || nqh != nkvh * GQA || n_pages < 1 || max_pages < 1 ||
      max_seq_len < T || max_seq_len > max_pages * Q27B_PAGE || B > 65535)
    return fail(Q27B_BAD_SHAPE, "attn_decode_paged: bad shape");
  if (!qn || !qg || !kpool || !vpool || !page_table || !seq_len || !o)
    return fail(Q27B_BAD_SHAPE, "attn_decode_paged: null pointer");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  // Fixed chunk length (a multiple of the page): about 8 chunks per SM over the whole batch at
  // the longest length, between 1024 and 8192 positions.
  const int64_t total = (int64_t)B * nkvh * max_seq_len;
  int chunk = (int)std::min<int64_t>(8192, std::max<int64_t>(1024, total / (8 * (int64_t)ctx->n_sm)));
  // The default kernel runs a batch as CTAs of one tile group, two per SM (the prologue and epilogue of one
  // overlap the streaming of the other), each with half the positions (Q27B_PAGED_GROUPS=2: one CTA of two
  // groups per SM, as for a single sequence).
  static const bool two_groups = [] {
    const char* e = getenv("Q27B_PAGED_GROUPS");
    return e && e[0] == '2';
  }();
  const int kc = kernel_choice();
  const bool single_group = (kc == 0 || kc == 3) && !two_groups;
  if (single_group) chunk = std::max(1024, chunk / 2);
  if (const char* e = getenv("Q27B_PAGED_CHUNK")) {  // tuning: chunk length in positions
    if (atoi(e) >= Q27B_PAGE) chunk = atoi(e);
  }
  chunk = (chunk + Q27B_PAGE - 1) / Q27B_PAGE * Q27B_PAGE;
  const int nch = (max_seq_len + chunk - 1) / chunk;
  float* part;
  if (int rc = paged_ws(ctx, (size_t)B * nkvh * nch * MAXR * PROW, &part)) return rc;
  // One pool = n_pages * nkvh pages of 256 rows: the same row tensor as a cache of that many rows.
  const int pool_rows_per_head = n_pages * Q27B_PAGE;
  CUtensorMap kvm, ksm, vvm, vsm;
  if (int rc = get_tmaps(kpool, nkvh, pool_rows_per_head, true, &kvm, &ksm)) return rc;
  if (int rc = get_tmaps(vpool, nkvh, pool_rows_per_head, true, &vvm, &vsm)) return rc;
  const CUtensorMap *kv = &kvm, *ks = &ksm, *vv = &vvm, *vs = &vsm;
  DecodeParams p = {};
  p.qn = qn; p.part = part; p.status = ctx->status;
  p.T = T; p.nqh = nqh; p.nkvh = nkvh; p.n_ctx = max_pages * Q27B_PAGE; p.nch = nch; p.kq_scale = kq_scale;
  p.base_pos = 0; p.n_local = -1;
  p.page_table = page_table; p.seq_len = seq_len; p.max_pages = max_pages; p.n_pages = n_pages; p.chunk_len = chunk;
  if (int rc = launch_q8(kv, ks, vv, vs, p, true, B, (cudaStream_t)stream, single_group)) return rc;
  MergeParams mp = {};
  mp.part = part; mp.nparts = nch; mp.rows = (int64_t)B * T * nqh; mp.qg = qg; mp.o = o; mp.T = T; mp.nqh = nqh;
  mp.seq_len = seq_len; mp.chunk_len = chunk;
  return launch_merge(mp, true, (cudaStream_t)stream);
}

}  // extern "C"
