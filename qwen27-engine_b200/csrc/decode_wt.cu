// Split-K flash-decode over a q8_0 KV cache: the warp-specialised kernel of decode_ws.cu with its second
// contraction, O += P V, moved to the 5th-generation tensor cores (tcgen05, accumulator in tensor memory).
//
// Same operator, decomposition, tile schedule and roundings as decode_ws.cu (attn_mma_kernel and the
// host wrapper attn_decode of the reference, src/attn.cu:95-292,894-918; roundings src/attn.cu:10-11).
// What changes is the P V half:
//
//   warps 0-3, 4-7    "QK" groups 0 and 1, as in decode_ws.cu: K tile -> S^T = K Q^T on warp MMAs with the
//                     int8 -> f16 conversion in registers -> P (f16). P goes into shared memory in the
//                     K-major, 128-byte-swizzled layout of a tcgen05 A operand ([query row][64 positions]),
//                     and one lane of the group issues the tile's four tcgen05.mma (128 x 256 x 16: the 24
//                     query rows on the M axis, the 256 head dims on N, 16 positions per instruction).
//   warps 8-11, 12-15 "CV" groups 0 and 1: V tile -> f16(q * d) into shared memory as the B operand
//                     ([16 positions][256 dims] chunks, MN-major, 128-byte swizzle: no transposition, which
//                     the warp-MMA form pays a byte shuffle per value for), three chunks in flight per group.
//                     No MMAs, no P fragments, no accumulators: 280 instructions per tile and warp where
//                     the P V warps of decode_ws.cu issue 460.
//   tensor memory     O of group g: lanes 0..23 (the query rows), columns 256 g .. 256 g + 255, f32.
//
// The legacy tensor pipe (8 cycles per m16n8k16 and scheduler, 44 % busy in decode_ws.cu and its most
// contended unit) carries only the S^T half; the P V half runs on the otherwise idle tcgen05 pipe.
// Shared memory pays for the f16 V chunks with shallower rings: two K and two V tiles in flight per group.
//
// The rare rescale of O (the group's reference maxima moved) is done in tensor memory by the group's
// first warp (lanes = rows) after the MMAs issued so far have completed. Every wait is bounded.
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
constexpr int NVF = 3;                            // f16 V chunks (16 positions) in flight per group
constexpr int VF_BYTES = 16 * 2 * AD;             // one chunk: [4 x 64 dims][16 positions][128 B]
constexpr int P_BYTES = MAXR * 128;               // one P tile: 24 rows x 64 positions f16
constexpr int Q_STRIDE = 2 * AD + 16;             // bytes per staged Q row (f16; padding: conflict-free 16-byte reads)
// shared memory map (offsets from a 1024-byte aligned base). The P tiles come first: as the A operand of an
// M = 128 MMA a tile is read 128 rows deep, and the 104 rows behind its 24 must be mapped memory (what they
// hold does not matter: they only reach accumulator rows that nobody reads).
constexpr int OFF_P = 0;                                       // [2 groups][2 buffers] P tiles
constexpr int OFF_Q = OFF_P + 4 * P_BYTES;                     // the staged Q block [24][Q_STRIDE]
constexpr int OFF_VF = (OFF_Q + MAXR * Q_STRIDE + 1023) / 1024 * 1024;  // [2 groups][NVF] f16 V chunks
constexpr int OFF_KRING = OFF_VF + 2 * NVF * VF_BYTES;         // [KDEPTH][2 groups] raw K tiles
constexpr int OFF_VRING = OFF_KRING + 2 * KDEPTH * HALF_BYTES; // [VDEPTH][2 groups] raw V tiles
constexpr int OFF_MAX = OFF_VRING + 2 * VDEPTH * HALF_BYTES;   // [2 groups][2 buffers][4 warps][24] floats
constexpr int OFF_F = OFF_MAX + 2 * 2 * 4 * MAXR * 4;          // [2 groups][24] floats: rescale factors
constexpr int OFF_L = OFF_F + 2 * MAXR * 4;                    // [2 groups][4 warps][24] floats: row sums at the end
constexpr int OFF_M1 = OFF_L + 2 * 4 * MAXR * 4;               // [2 groups][24] floats: reference maxima at the end
constexpr int OFF_BAR = OFF_M1 + 2 * MAXR * 4;                 // mbarriers, see the enum
constexpr int NBAR = 32;
constexpr int OFF_FLAG = OFF_BAR + NBAR * 8;                   // abort flag, tensor-memory base address
constexpr int OFF_TOK = OFF_FLAG + 16;                         // [2 groups][2 buffers] words: "move the maxima" tokens
constexpr int OFF_SEQ = OFF_TOK + 16;                          // [2 groups][8] ints: the groups' tile queues
constexpr int SMEM_USED = OFF_SEQ + 64;
constexpr int WT_SMEM_BYTES = SMEM_USED + 1024;                // slack for the 1024-byte alignment
constexpr int O_STRIDE = AD + 4;                               // floats per row of the end-of-kernel O exchange
static_assert(OFF_VF % 1024 == 0 && VF_BYTES % 1024 == 0 && P_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
static_assert(OFF_KRING % 1024 == 0 && HALF_BYTES % 1024 == 0, "TMA tiles need 1024-byte alignment");
static_assert(OFF_P + 3 * P_BYTES + 128 * 128 <= SMEM_USED, "an A operand is read 128 rows deep");
static_assert(2 * MAXR * O_STRIDE * 4 <= 2 * KDEPTH * HALF_BYTES, "O exchange must fit in the K ring");
static_assert(WT_SMEM_BYTES <= 232448, "shared memory budget of one CTA");

// mbarrier indices
enum {
  B_KFULL = 0,                 // [2 * KDEPTH] raw K tile landed (TMA)
  B_VFULL = B_KFULL + 2 * KDEPTH,  // [2 * VDEPTH] raw V tile landed (TMA)
  B_VFFULL = B_VFULL + 2 * VDEPTH, // [2 groups][NVF] f16 V chunk written (4 converter warps)
  B_VFFREE = B_VFFULL + 2 * NVF,   // [2 groups][NVF] the chunk's MMA has completed
  B_PFREE = B_VFFREE + 2 * NVF,    // [2 groups][2] the MMAs that read this P tile have completed
  B_ODONE = B_PFREE + 4,           // [2 groups] every MMA of the group has completed
  B_COUNT = B_ODONE + 2,
};
static_assert(B_COUNT <= NBAR, "barrier table");

constexpr float TAU = 8.0f;                           // a score may exceed the reference max by this much
constexpr int WT_THREADS = 512;
constexpr uint32_t IDESC_PV = umma_idesc(1, 0, 0, 0, 1, 128, AD);  // f32 += f16 * f16, A K-major, B MN-major, M128 N256
// Named barriers (0 is __syncthreads).
constexpr int BAR_QK = 1;      // + group: the four QK warps of a group
constexpr int BAR_CV = 3;      // + group: the four converter warps of a group

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
    for (int s = 0; s < 2 * NVF; s++) {
      mbar_init(&bar[B_VFFULL + s], 4);
      mbar_init(&bar[B_VFFREE + s], 1);
    }
    for (int s = 0; s < 4; s++) mbar_init(&bar[B_PFREE + s], 1);
    mbar_init(&bar[B_ODONE], 1);
    mbar_init(&bar[B_ODONE + 1], 1);
    *abort_flag = 0;
    for (int i = 0; i < 4; i++) ((volatile uint32_t*)(sgen + OFF_TOK))[i] = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

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
  // Only the loader of a QK group asks; everybody else reads the answer from the queue in shared
  // memory (8 entries per group, entry j mod 8), which the loader fills two tiles ahead.
  auto next_tile = [&](int j) {
    const int i = grp + 2 * j;
    if (i < n_static) return t_first + i;
    if (!has_pool) return -1;
    const int t = pool0 + atomicAdd(p.sched + kh, 1);
    return t < ntiles_all ? t : -1;
  };
  const uint32_t sSeq = sbase + OFF_SEQ + grp * 32;

  const bool is_qk = warp < 8;
  const bool loader = wq == 0 && lane == 0;  // refills this group's raw K (QK warps) or raw V (CV warps) tiles
  int pend = -1;  // QK loader: the tile that goes into the queue next
  if (loader && is_qk) {
    const int t0 = next_tile(0);
    sts32(sSeq + 0, (uint32_t)t0);
    if (t0 >= 0) issue_k(t0, 0);
    const int t1 = t0 < 0 ? -1 : next_tile(1);
    sts32(sSeq + 4, (uint32_t)t1);
    if (t1 >= 0) issue_k(t1, 1);
    pend = t1 < 0 ? -1 : next_tile(2);
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
  if (loader && !is_qk) {
    const int t0 = (int)lds32(sSeq + 0), t1 = (int)lds32(sSeq + 4);
    if (t0 >= 0) issue_v(t0, 0);
    if (t1 >= 0) issue_v(t1, 1);
  }
  const uint32_t MAGIC = 0x64646464u;

  if (is_qk) {
    // ======================================================================== QK warps
    const uint32_t sQl = sbase + OFF_Q + g * Q_STRIDE + 32 * tg;
    const uint32_t sPg = sbase + OFF_P + grp * 2 * P_BYTES;
    const uint32_t sF = sbase + OFF_F + grp * MAXR * 4;
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
    const uint32_t pA = slot_row(g) * 2;
    int nmma = 0;  // issuing lane: 16-position chunks issued so far

    for (int jt = 0;; jt++) {
      const int tile = (int)lds32(sSeq + (jt & 7) * 4);
      if (tile < 0) break;
      const int s = 2 * (jt % KDEPTH) + grp;
      mbar_wait(&bar[B_KFULL + s], (jt / KDEPTH) & 1, abort_flag, p.status);
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
      if (jt >= 2) mbar_wait(&bar[B_PFREE + 2 * grp + buf], ((jt >> 1) - 1) & 1, abort_flag, p.status);
      const uint32_t sPt = sPg + buf * P_BYTES;
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const int r = 8 * nt + 2 * tg + e;
          sts16(sPt + r * 128 + (((2 * wq) ^ (r & 7)) << 4) + pA, pw[nt][e] & 0xffffu);
          sts16(sPt + r * 128 + (((2 * wq + 1) ^ (r & 7)) << 4) + pA, pw[nt][e] >> 16);
        }
      fence_proxy_async();  // the tile is read by the tensor core
      bar_sync(BAR_QK + grp, 128);
      // All four warps have read this raw K tile: refill its buffer with the group's tile jt + 2, and ask
      // for the one after that.
      if (loader) {
        sts32(sSeq + ((jt + 2) & 7) * 4, (uint32_t)pend);
        if (pend >= 0) {
          issue_k(pend, jt + 2);
          pend = next_tile(jt + 3);
        }
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
            if (wq == 0 && g == 0) stsf(sF + r * 4, f);
            const float mb = mn * LOG2E;
            const float pa = ex2(fmaf(sacc[nt][e], LOG2E, -mb)), pb = ex2(fmaf(sacc[nt][2 + e], LOG2E, -mb));
            lt[nt][e] = pa + pb;
            sts16(sPt + r * 128 + (((2 * wq) ^ (r & 7)) << 4) + pA, pack_h2(pa, pb) & 0xffffu);
            sts16(sPt + r * 128 + (((2 * wq + 1) ^ (r & 7)) << 4) + pA, pack_h2(pa, pb) >> 16);
          }
        fence_proxy_async();
        if (jt > 0 && wq == 0) {
          // O of this group holds the tiles before jt, scaled to the old maxima: once the MMAs of the
          // previous tile have completed, the group's first warp (lane = query row) multiplies its rows.
          __syncwarp();
          mbar_wait(&bar[B_PFREE + 2 * grp + (buf ^ 1)], ((jt - 1) >> 1) & 1, abort_flag, p.status);
          tc_fence_after();
          __syncwarp();  // (the factors of all rows are in shared memory: written by this warp's lanes above)
          const float f = lane < MAXR ? ldsf(sF + lane * 4) : 1.f;
#pragma unroll 1
          for (int c = 0; c < AD / 32; c++) {
            uint32_t v[32];
            tmem_ld32(tmem + grp * AD + c * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
            tmem_st32(tmem + grp * AD + c * 32, v);
          }
          tc_wait_st();
          tc_fence_before();
        }
        bar_sync(BAR_QK + grp, 128);
      }
      // ---- the tile's four MMAs, O (+)= P[24 x 16 positions] V[16 positions x 256], issued by one lane
      if (loader) {
        tc_fence_after();
#pragma unroll 1
        for (int kk = 0; kk < 4; kk++, nmma++) {
          const int sl = nmma % NVF;
          mbar_wait(&bar[B_VFFULL + grp * NVF + sl], (nmma / NVF) & 1, abort_flag, p.status);
          tc_fence_after();
          if (*abort_flag) break;
          const uint64_t da = umma_desc_sw128(sPt + kk * 32, 16, 1024);
          const uint64_t db = umma_desc_sw128(sbase + OFF_VF + (grp * NVF + sl) * VF_BYTES, 16 * 128, 1024);
          tc_mma_f16(tmem + grp * AD, da, db, IDESC_PV, (jt > 0 || kk > 0) ? 1u : 0u);
          tc_commit(&bar[B_VFFREE + grp * NVF + sl]);
        }
        tc_commit(&bar[B_PFREE + 2 * grp + buf]);
      }
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        l[nt][0] += lt[nt][0];
        l[nt][1] += lt[nt][1];
      }
    }
    if (loader) tc_commit(&bar[B_ODONE + grp]);

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
    int nconv = 0;  // 16-position chunks converted so far
    for (int jt = 0;; jt++) {
      const int tile = (int)lds32(sSeq + (jt & 7) * 4);
      if (tile < 0) break;
      const int s = 2 * (jt % VDEPTH) + grp;
      const uint32_t st = sbase + OFF_VRING + s * HALF_BYTES;
      const int tile_p0 = tile * TILE;
      mbar_wait(&bar[B_VFULL + s], (jt / VDEPTH) & 1, abort_flag, p.status);
#pragma unroll 1
      for (int kk = 0; kk < 4; kk++, nconv++) {
        const int sl = nconv % NVF;
        if (nconv >= NVF) mbar_wait(&bar[B_VFFREE + grp * NVF + sl], ((nconv / NVF) - 1) & 1, abort_flag, p.status);
        const uint32_t vf = sbase + OFF_VF + (grp * NVF + sl) * VF_BYTES;
        uint4 x[2];
        uint32_t d[2];
#pragma unroll
        for (int k = 0; k < 2; k++) {
          x[k] = lds128(st + cv_src + (2 * kk + k) * 1024);
          d[k] = ldsu16(st + cv_sc + (2 * kk + k) * 128);
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {
          // rows past the end of the sequence may hold anything: P is 0 there, V must be too
          if (tile_p0 + 16 * kk + 8 * k + cv_row0 >= n_end) d[k] = 0, x[k] = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
          const __half2 dd = u32_as_h2(prmt(d[k], d[k], 0x1010));
          const uint32_t xw[4] = {x[k].x ^ 0x80808080u, x[k].y ^ 0x80808080u, x[k].z ^ 0x80808080u, x[k].w ^ 0x80808080u};
          uint32_t o[8];
#pragma unroll
          for (int w = 0; w < 4; w++) {
            o[2 * w] = dq_pair(prmt(xw[w], MAGIC, 0x4140), dd);
            o[2 * w + 1] = dq_pair(prmt(xw[w], MAGIC, 0x4342), dd);
          }
          const uint32_t dst = vf + cv_dst + k * 1024;
          sts128(dst, o[0], o[1], o[2], o[3]);
          sts128(dst ^ 16u, o[4], o[5], o[6], o[7]);
        }
        fence_proxy_async();  // the chunk is read by the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[B_VFFULL + grp * NVF + sl]);
      }
      // Every converter warp of the group has read this raw V tile: refill its buffer with the group's tile
      // jt + 2 (the queue entry was written before the QK group released tile jt).
      // (That entry is in place: this tile's last chunk could only be converted after the first MMA of the
      // tile had completed, and the QK loader writes the entry before it issues that MMA.)
      bar_sync(BAR_CV + grp, 128);
      if (loader) {
        const int tn = (int)lds32(sSeq + ((jt + 2) & 7) * 4);
        if (tn >= 0) issue_v(tn, jt + 2);
      }
    }
  }
  __syncthreads();  // every tile consumed: the rings are free for the O exchange; m and l are posted

  // ---- O out of tensor memory: rows = lanes 0..23 of the quarter that warps 0, 4, 8, 12 may read; warp 4 w
  // reads columns 128 (w & 1) .. +127 of group w >> 1, scales them to the common maxima and adds them up
  // through shared memory.
  const uint32_t sO = sbase + OFF_KRING;  // [2 halves... see below] f32 [24][O_STRIDE]
  if (wq == 0) {
    const int og = warp >> 3, oh = (warp >> 2) & 1;  // group whose O this warp reads, and which half of its columns
    mbar_wait(&bar[B_ODONE + og], 0, abort_flag, p.status);
    tc_fence_after();
    float f = 0.f;
    if (lane < R) {
      const float m0 = ldsf(sbase + OFF_M1 + lane * 4), m1 = ldsf(sbase + OFF_M1 + (MAXR + lane) * 4);
      const float M = fmaxf(m0, m1);
      f = ex2(((og ? m1 : m0) - M) * LOG2E);
      // a group without tiles never issued an MMA: its accumulator is not initialised
      if ((og ? m1 : m0) <= M_INIT) f = 0.f;
    }
#pragma unroll 1
    for (int c = 0; c < 4; c++) {
      uint32_t v[32];
      tmem_ld32(tmem + og * AD + oh * 128 + c * 32, v);
      tc_wait_ld();
      if (lane < R) {
#pragma unroll
        for (int i = 0; i < 32; i++) {
          const float x = f == 0.f ? 0.f : __uint_as_float(v[i]) * f;
          stsf(sO + ((og * MAXR + lane) * O_STRIDE + oh * 128 + c * 32 + i) * 4, x);
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
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
  if (has_pool && tid == 0) {
    // Both loaders of this CTA have drawn their last pool tile. The last CTA of the grid to say so
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
    tmem_dealloc(tmem, 512);
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
