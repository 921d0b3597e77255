// Split-K flash-decode over a q8_0 KV cache with both contractions on the 5th-generation tensor
// cores (tcgen05.mma kind::f16, accumulators in TMEM).
//
// Same operator, same work decomposition, same partial layout and same roundings as the warp-MMA
// kernel in decode.cu (reference: attn_mma_kernel, src/attn.cu:95-292): Q * scale -> f16,
// K / V -> f16(int8 * f16 scale), P -> f16, f32 accumulation, row sums from the f32 P.
// Why a second kernel: measured on B200, the legacy mma.sync path shares its issue bandwidth with
// the int8 -> f16 conversion arithmetic, so the warp-MMA kernel is bound by instruction issue. Here
// the SIMT lanes only dequantise and do the softmax; the contractions are asynchronous hardware.
// Two measured properties of tcgen05.mma shape the design: an MMA costs time in proportion to its
// A operand (about 54 cycles per 128 x 16 f16 block, whatever N is), and operands read from shared
// memory compete with TMA writes and converter traffic for the 128 B per clock of the SM. So the
// large streamed operand goes where it is cheapest:
//
//   S^T = K Q^T   K (128 positions x 256 dims, f16) is the A operand and lives in TMEM: the K
//                 converters store their f16 values straight into TMEM and K never returns to
//                 shared memory. Q^T (32 rows) is the small B operand in shared memory.
//   O   = P V     P (query rows x 128 positions, f16) is the A operand in TMEM; V (f16, shared
//                 memory, [64-dim segment][position][128 B], 128-byte swizzle) is the B operand
//                 read "MN-major": four MMAs of N = 256 per 64 positions.
//
// Warps: 0-7 K converters (warp w: TMEM lane quarter w % 4 = 32 positions, dims 128 (w / 4) ..+127),
// 8-15 V converters, 16-19 softmax (a thread owns one position of the tile: S^T row from TMEM,
// P = exp(S - m) against reference maxima kept in shared memory and moved only when a score exceeds
// them by more than TAU, per-lane partial row sums), 20 "mover" (lanes = query rows: transposes P
// from the softmax staging buffer into TMEM, rescales O when the maxima moved, writes the partial),
// 21 TMA producer, 22 issuer of the first MMA (owns the TMEM allocation), 23 issuer of the second.
// Raw data arrives in 17 KB items (K or V of 64 positions: int8 values + f16 scales) through one
// ring of seven slots, K two tiles ahead of V, so that S^T of a tile is ready long before its V.
// TMEM columns: 0-127 K (two halves of 64, each recycled as soon as its eight MMAs have completed),
// 128-191 two S^T buffers, 192-255 P, 256-511 O.
#include "common.cuh"
#include "decode_params.h"

namespace q27b {
namespace {

constexpr int SUB = 64;                     // positions per raw item
constexpr int TILE = 128;                   // positions per tile (two items of K, two of V)
constexpr int NSLOT = 7;                    // raw ring slots
constexpr int SEG = SUB * 128;              // [64 positions][128 B]
constexpr int ITEM_BYTES = 2 * SEG + SUB * 16;      // 17408: int8 values (two halves of 128 dims) + f16 scales
constexpr int I_SC = 2 * SEG;
constexpr int VF_BYTES = 4 * SEG;           // f16 V of 64 positions, 32 KB
constexpr int QSEG = 32 * 128;              // one 64-dim segment of Q^T: [32 rows][128 B]
constexpr int PS_ROW = 2 * TILE + 16;       // staging row of P: 128 f16 + padding (bank spread)
constexpr int PS_BYTES = MAXR * PS_ROW;     // 6528
constexpr int OFF_RAW = 0;
constexpr int OFF_VF = OFF_RAW + NSLOT * ITEM_BYTES;   // two buffers; reused to stage the partial at the end
constexpr int OFF_Q = OFF_VF + 2 * VF_BYTES;
constexpr int OFF_PS = OFF_Q + 4 * QSEG;               // two buffers
constexpr int OFF_X = OFF_PS + 2 * PS_BYTES;           // floats
constexpr int X_M = 0, X_F = 24, X_CMAX = 72, X_L = 168, X_TOK = 264;  // m[24], f[2][24], colmax[4][24], l[4][24], token[2]
constexpr int OFF_BAR = OFF_X + 272 * 4;
enum {
  B_RAWFULL = 0,     // [7]
  B_RAWEMPTY = 7,    // [7]
  B_KTFULL = 14,     // [2] K half in TMEM
  B_KTEMPTY = 16,    // [2]
  B_VFFULL = 18,     // [2]
  B_VFEMPTY = 20,    // [2]
  B_SFULL = 22,      // [2]
  B_SEMPTY = 24,     // [2]
  B_PSFULL = 26,     // [2] P staged in shared memory
  B_PSEMPTY = 28,    // [2]
  B_PTFULL = 30,     // P in TMEM
  B_PTEMPTY = 31,
  B_QFULL = 32,
  B_ODONE = 33,
  NBAR = 34,
};
static_assert(NSLOT == 7, "barrier numbering assumes seven raw slots");
constexpr int OFF_MISC = OFF_BAR + NBAR * 8;
constexpr int TC_SMEM_USED = OFF_MISC + 16;
constexpr int TC_SMEM_BYTES = TC_SMEM_USED + 1024;
static_assert(OFF_VF % 1024 == 0 && OFF_Q % 1024 == 0 && ITEM_BYTES % 1024 == 0, "swizzled tiles need 1024-byte alignment");
static_assert(OFF_PS % 16 == 0 && OFF_X % 16 == 0 && OFF_BAR % 8 == 0, "alignment");
static_assert(TC_SMEM_BYTES <= 232448, "shared memory budget of one CTA");
static_assert(MAXR * PROW * 4 <= 2 * VF_BYTES, "partial staging fits the V buffers");

constexpr int KW0 = 0, VW0 = 8, SM_WARP0 = 16, MOVER_WARP = 20, TMA_WARP = 21, QK_WARP = 22, PV_WARP = 23;
constexpr int TC_THREADS = 24 * 32;
constexpr int BAR_SM = 1;                   // named barrier of the softmax group (128 threads)
constexpr int BAR_OUT = 2;                  // softmax group + mover (160 threads)
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_K = 0, TM_S = 128, TM_P = 192, TM_O = 256;
constexpr float TAU = 8.0f;
constexpr uint32_t IDESC_QK = umma_idesc(1, 0, 0, 0, 0, 128, 32);   // f32 += f16 * f16, A (TMEM) and B K-major, M128 N32
constexpr uint32_t IDESC_PV = umma_idesc(1, 0, 0, 0, 1, 128, 256);  // A (TMEM) K-major, B (V) MN-major, M128 N256

__device__ __forceinline__ void sm_sync() { asm volatile("bar.sync %0, 128;" ::"r"(BAR_SM) : "memory"); }
__device__ __forceinline__ void out_sync() { asm volatile("bar.sync %0, 160;" ::"r"(BAR_OUT) : "memory"); }

// Position of the raw items in the ring's sequence: K(0), K(1), then V(j), K(j + 2) for j = 0, 1, ...
// (each tile has two items, s = 0, 1).
__device__ __forceinline__ int k_item(int j, int s) { return j < 2 ? 2 * j + s : 4 * j - 2 + s; }
__device__ __forceinline__ int v_item(int j, int s) { return 4 * j + 4 + s; }

// 16 int8 (one 16-byte chunk, biased to unsigned by the caller's xor) -> 16 f16 = 8 words.
__device__ __forceinline__ void dq16(const uint4 x, const __half2 dd, uint32_t* o) {
  const uint32_t xw[4] = {x.x ^ 0x80808080u, x.y ^ 0x80808080u, x.z ^ 0x80808080u, x.w ^ 0x80808080u};
#pragma unroll
  for (int w = 0; w < 4; w++) {
    o[2 * w] = dq_pair(__byte_perm(xw[w], 0x64646464u, 0x4140), dd);
    o[2 * w + 1] = dq_pair(__byte_perm(xw[w], 0x64646464u, 0x4342), dd);
  }
}

template <bool PAGED>
__global__ void __launch_bounds__(TC_THREADS, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_ks,
                 const __grid_constant__ CUtensorMap tm_vv, const __grid_constant__ CUtensorMap tm_vs,
                 const DecodeParams p) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  uint64_t* bar = (uint64_t*)(sgen + OFF_BAR);
  uint32_t* tmem_slot = (uint32_t*)(sgen + OFF_MISC);
  volatile int* abort_flag = (volatile int*)(sgen + OFF_MISC + 4);
  float* xf = (float*)(sgen + OFF_X);
  volatile uint32_t* tok = (volatile uint32_t*)(xf + X_TOK);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ch = blockIdx.x, kh = blockIdx.y;
  const int T = p.T, R = GQA * T;
  const int seq = PAGED ? blockIdx.z : 0;
  const int pos0 = PAGED ? p.seq_len[seq] - T : *p.pos0;
  const float* qn = p.qn + (size_t)seq * T * p.nqh * AD;

  // Local rows to attend, and this CTA's chunk [c0, c1) of them (chunk starts are multiples of SUB).
  int n = pos0 + T - p.base_pos;
  if (p.n_local >= 0) n = min(n, p.n_local);
  n = max(0, min(n, p.n_ctx));
  int chunk;
  if (PAGED) {
    chunk = p.chunk_len;
  } else {
    chunk = (n + p.nch - 1) / p.nch;
    chunk = max(SUB, (chunk + SUB - 1) / SUB * SUB);
  }
  const int c0 = min(n, ch * chunk), c1 = min(n, c0 + chunk);
  float* out = p.part + (((size_t)seq * p.nkvh + kh) * p.nch + ch) * MAXR * PROW;
  if (c0 >= c1) {  // empty chunk: neutral partial (src/attn.cu:117-120); the paged merge never reads it
    if (!PAGED)
      for (int i = tid; i < R * PROW; i += TC_THREADS) out[i] = (i % PROW == 0) ? M_INIT : 0.f;
    return;
  }
  const int nsub = (c1 - c0 + SUB - 1) / SUB;  // raw items of K (and of V)
  const int nt = (nsub + 1) / 2;               // tiles; the last one may have one item only

  if (tid == 0) {
    for (int s = 0; s < NSLOT; s++) {
      mbar_init(&bar[B_RAWFULL + s], 1);
      mbar_init(&bar[B_RAWEMPTY + s], 8);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(&bar[B_KTFULL + s], 4);
      mbar_init(&bar[B_KTEMPTY + s], 1);
      mbar_init(&bar[B_VFFULL + s], 8);
      mbar_init(&bar[B_VFEMPTY + s], 1);
      mbar_init(&bar[B_SFULL + s], 1);
      mbar_init(&bar[B_SEMPTY + s], 4);
      mbar_init(&bar[B_PSFULL + s], 4);
      mbar_init(&bar[B_PSEMPTY + s], 1);
    }
    mbar_init(&bar[B_PTFULL], 1);
    mbar_init(&bar[B_PTEMPTY], 1);
    mbar_init(&bar[B_QFULL], 4);
    mbar_init(&bar[B_ODONE], 1);
    *abort_flag = 0;
    tok[0] = 0;
    tok[1] = 0;
    mbar_fence_init();
  }
  if (tid < MAXR) xf[X_M + tid] = M_INIT;
  if (warp == QK_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < VW0) {
    // ================================================================ K converters: raw item -> TMEM
    const int kq = warp & 3, kh2 = warp >> 2;
    const int ksub = kq >> 1, krow = (kq & 1) * 32 + lane;
    const uint32_t ktaddr = tmem + ((uint32_t)(kq * 32) << 16) + TM_K + kh2 * 64;
    _Pragma("unroll 1") for (int j = 0; j < nt && !*abort_flag; j++) {
      mbar_wait(&bar[B_KTEMPTY + kh2], (j & 1) ^ 1, abort_flag, p.status);
      if (2 * j + ksub < nsub) {
        const int item = k_item(j, ksub), slot = item % NSLOT;
        const uint8_t* raw = sgen + OFF_RAW + slot * ITEM_BYTES;
        mbar_wait(&bar[B_RAWFULL + slot], (item / NSLOT) & 1, abort_flag, p.status);
        const uint8_t* vals = raw + kh2 * SEG;
        const uint2 sc = *(const uint2*)(raw + I_SC + krow * 16 + kh2 * 8);
        // All loads first: the compiler cannot move a shared-memory load above an earlier store or
        // TMEM store, so interleaving them would serialise the load latencies.
        uint4 x[8];
#pragma unroll
        for (int c = 0; c < 8; c++) x[c] = *(const uint4*)(vals + swz128(krow, c));
        tc_fence_after();
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
          uint32_t o[32];
          const __half2 d0 = __half2half2(__ushort_as_half((unsigned short)((hh ? sc.y : sc.x) & 0xffffu)));
          const __half2 d1 = __half2half2(__ushort_as_half((unsigned short)((hh ? sc.y : sc.x) >> 16)));
#pragma unroll
          for (int c = 0; c < 4; c++) dq16(x[hh * 4 + c], c < 2 ? d0 : d1, o + 8 * c);
          tmem_st32(ktaddr + hh * 32, o);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_n(&bar[B_RAWEMPTY + slot], 2);  // four warps share an item
      }
      if (lane == 0) mbar_arrive(&bar[B_KTFULL + kh2]);
    }
  } else if (warp < SM_WARP0) {
    // ================================================================ V converters: raw item -> f16 tile
    // One unit = 16 int8 of one row -> 16 f16 (two 16-byte chunks of a segment row). Eight
    // neighbouring lanes take 4 units of rows rho and rho ^ 5, which keeps the swizzled 16-byte loads
    // and stores free of bank conflicts. 1024 units per item, 4 per thread.
    const int vt = tid - VW0 * 32;
    int it_row[4], it_c16[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int u = vt + 256 * k;
      it_row[k] = (2 * (u >> 5)) ^ (5 * ((u >> 2) & 1));
      it_c16[k] = (u & 3) + 4 * ((u >> 3) & 3);
    }
    _Pragma("unroll 1") for (int g = 0; g < nsub && !*abort_flag; g++) {
      const int j = g >> 1, s = g & 1;
      const int item = v_item(j, s), slot = item % NSLOT;
      const uint8_t* raw = sgen + OFF_RAW + slot * ITEM_BYTES;
      uint8_t* dst = sgen + OFF_VF + s * VF_BYTES;
      const int rows_valid = c1 - (c0 + g * SUB);
      mbar_wait(&bar[B_RAWFULL + slot], (item / NSLOT) & 1, abort_flag, p.status);
      mbar_wait(&bar[B_VFEMPTY + s], (j & 1) ^ 1, abort_flag, p.status);
      uint4 x[4];
      __half d[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {  // loads first (a load cannot be moved above an earlier shared-memory store)
        const int row = it_row[k], c16 = it_c16[k];
        x[k] = *(const uint4*)(raw + (c16 >> 3) * SEG + swz128(row, c16 & 7));
        d[k] = *(const __half*)(raw + I_SC + row * 16 + (c16 >> 1) * 2);
      }
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const int row = it_row[k], c16 = it_c16[k];
        uint32_t o[8];
        dq16(x[k], __half2half2(d[k]), o);
        if (row >= rows_valid) {  // rows past the end may hold anything: P is 0 there, V must be too
#pragma unroll
          for (int w = 0; w < 8; w++) o[w] = 0;
        }
        uint8_t* seg = dst + (c16 >> 2) * SEG;
        const uint32_t cc = 2 * (c16 & 3);
        *(uint4*)(seg + swz128(row, cc)) = make_uint4(o[0], o[1], o[2], o[3]);
        *(uint4*)(seg + swz128(row, cc + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bar[B_VFFULL + s]);
        mbar_arrive(&bar[B_RAWEMPTY + slot]);
      }
    }
  } else if (warp < MOVER_WARP) {
    // ================================================================ softmax group
    const int sw = warp - SM_WARP0;          // TMEM lane quarter
    const int st_tid = tid - SM_WARP0 * 32;  // 0..127 = position within the tile = TMEM lane
    const uint32_t tlane = tmem + ((uint32_t)(sw * 32) << 16);
    // Q^T (B operand of S^T = K Q^T): [4 segments][32 rows][128 B], scaled, f16; rows >= 6T are zero.
    {
      const int r = st_tid >> 2, sg = st_tid & 3;
      uint8_t* dst = sgen + OFF_Q + sg * QSEG;
#pragma unroll
      for (int c = 0; c < 8; c++) {
        uint32_t w[4] = {0, 0, 0, 0};
        if (r < R) {
          const float* src = qn + ((size_t)(r / GQA) * p.nqh + kh * GQA + r % GQA) * AD + sg * 64 + c * 8;
          const float4 a = *(const float4*)src, b = *(const float4*)(src + 4);
          w[0] = pack_h2(a.x * p.kq_scale, a.y * p.kq_scale);
          w[1] = pack_h2(a.z * p.kq_scale, a.w * p.kq_scale);
          w[2] = pack_h2(b.x * p.kq_scale, b.y * p.kq_scale);
          w[3] = pack_h2(b.z * p.kq_scale, b.w * p.kq_scale);
        }
        *(uint4*)(dst + swz128(r, c)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_QFULL]);
    }

    float lacc[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; r++) lacc[r] = 0.f;
    const int lim_base = pos0 + 1 - p.base_pos;  // local rows < lim_base + t are visible to token t
    const int lim_min = min(c1, lim_base);       // positions below this are visible to every row

    _Pragma("unroll 1") for (int j = 0; j < nt; j++) {
      const int slot = j & 1;
      const int pos = c0 + j * TILE + st_tid;
      float s[MAXR];
      mbar_wait(&bar[B_SFULL + slot], (j >> 1) & 1, abort_flag, p.status);
      tc_fence_after();
      {
        uint32_t v[32];
        tmem_ld32(tlane + TM_S + slot * 32, v);
        tc_wait_ld();
#pragma unroll
        for (int r = 0; r < MAXR; r++) s[r] = __uint_as_float(v[r]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_SEMPTY + slot]);
      // The mover has finished with this slot's staging buffer, token and factors (tile j - 2).
      mbar_wait(&bar[B_PSEMPTY + slot], ((j >> 1) & 1) ^ 1, abort_flag, p.status);
      if (c0 + (j + 1) * TILE > lim_min) {  // edge tile: causal limit per token, end of the chunk, absent item
#pragma unroll
        for (int r = 0; r < MAXR; r++)
          if (pos >= min(c1, lim_base + min(r / GQA, T - 1))) s[r] = -INFINITY;
      }
      bool exceed = j == 0;
#pragma unroll
      for (int r = 0; r < MAXR; r++) exceed |= s[r] > xf[X_M + r] + TAU;
      if (__any_sync(0xffffffffu, exceed) && lane == 0) tok[slot] = (uint32_t)(j + 1);
      sm_sync();
      if (tok[slot] == (uint32_t)(j + 1)) {
        // ---- some score ran away from the reference maxima (always on the first tile): move them
#pragma unroll
        for (int r = 0; r < MAXR; r++) {
          float v = s[r];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
          if (lane == 0) xf[X_CMAX + sw * MAXR + r] = v;
        }
        sm_sync();
        if (st_tid < MAXR) {  // everybody compared against the old maxima before the first barrier of this tile
          const int r = st_tid;
          const float mo = xf[X_M + r];
          const float mn = fmaxf(fmaxf(mo, xf[X_CMAX + r]),
                                 fmaxf(fmaxf(xf[X_CMAX + MAXR + r], xf[X_CMAX + 2 * MAXR + r]), xf[X_CMAX + 3 * MAXR + r]));
          xf[X_F + slot * MAXR + r] = ex2((mo - mn) * LOG2E);  // the mover rescales O by it
          xf[X_M + r] = mn;
        }
        sm_sync();
#pragma unroll
        for (int r = 0; r < MAXR; r++) lacc[r] *= xf[X_F + slot * MAXR + r];
      }
      // P = exp(S - m): per-lane partial row sums; f16 P[r][position] staged for the mover
      uint8_t* ps = sgen + OFF_PS + slot * PS_BYTES + st_tid * 2;
#pragma unroll
      for (int g6 = 0; g6 < MAXR / 6; g6++) {  // maxima in batches: their loads cannot pass the stores of P
        float nm[6];
#pragma unroll
        for (int k = 0; k < 6; k++) nm[k] = -xf[X_M + g6 * 6 + k] * LOG2E;
#pragma unroll
        for (int k = 0; k < 6; k++) {
          const int r = g6 * 6 + k;
          const float e = ex2(fmaf(s[r], LOG2E, nm[k]));
          lacc[r] += e;
          *(__half*)(ps + r * PS_ROW) = __float2half_rn(e);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_PSFULL + slot]);
    }

    // ---- row sums over the 128 position lanes; then help the mover write the partial
#pragma unroll
    for (int r = 0; r < MAXR; r++) {
      float v = lacc[r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) xf[X_L + sw * MAXR + r] = v;
    }
    out_sync();  // row sums visible to the mover
    out_sync();  // partial staged
    const float* ost = (const float*)(sgen + OFF_VF);
    for (int i = st_tid; i < R * PROW; i += 160) out[i] = ost[i];
  } else if (warp == MOVER_WARP) {
    // ================================================================ mover (lanes = query rows)
    const bool row_ok = lane < MAXR;
    _Pragma("unroll 1") for (int j = 0; j < nt; j++) {
      const int slot = j & 1;
      mbar_wait(&bar[B_PSFULL + slot], (j >> 1) & 1, abort_flag, p.status);
      mbar_wait(&bar[B_PTEMPTY], (j & 1) ^ 1, abort_flag, p.status);  // second MMA of tile j - 1 complete
      tc_fence_after();
      if (j > 0 && tok[slot] == (uint32_t)(j + 1)) {
        const float f = row_ok ? xf[X_F + slot * MAXR + lane] : 1.f;
#pragma unroll 1
        for (int c = 0; c < 8; c++) {
          uint32_t v[32];
          tmem_ld32(tmem + TM_O + c * 32, v);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
          tmem_st32(tmem + TM_O + c * 32, v);
        }
      }
      const uint8_t* ps = sgen + OFF_PS + slot * PS_BYTES + (row_ok ? lane : 0) * PS_ROW;
#pragma unroll
      for (int hh = 0; hh < 2; hh++) {
        uint32_t w[32];
#pragma unroll
        for (int c = 0; c < 8; c++) {
          uint4 x = *(const uint4*)(ps + (hh * 8 + c) * 16);
          if (!row_ok) x = make_uint4(0, 0, 0, 0);
          w[4 * c] = x.x; w[4 * c + 1] = x.y; w[4 * c + 2] = x.z; w[4 * c + 3] = x.w;
        }
        tmem_st32(tmem + TM_P + hh * 32, w);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bar[B_PSEMPTY + slot]);
        mbar_arrive(&bar[B_PTFULL]);
      }
    }
    // ---- partial (m, l, O[256]) per query row, staged in shared memory and written by five warps
    out_sync();
    mbar_wait(&bar[B_ODONE], 0, abort_flag, p.status);
    tc_fence_after();
    float* ost = (float*)(sgen + OFF_VF);
    if (lane < R) {
      ost[lane * PROW] = xf[X_M + lane];
      ost[lane * PROW + 1] = (xf[X_L + lane] + xf[X_L + MAXR + lane]) + (xf[X_L + 2 * MAXR + lane] + xf[X_L + 3 * MAXR + lane]);
    }
#pragma unroll 1
    for (int c = 0; c < 8; c++) {
      uint32_t v[32];
      tmem_ld32(tmem + TM_O + c * 32, v);
      tc_wait_ld();
      if (lane < R) {
#pragma unroll
        for (int i = 0; i < 32; i++) ost[lane * PROW + 2 + c * 32 + i] = __uint_as_float(v[i]);
      }
    }
    tc_fence_before();
    out_sync();
    for (int i = 128 + lane; i < R * PROW; i += 160) out[i] = ost[i];
  } else if (warp == TMA_WARP) {
    // ================================================================ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_kv);
      tma_prefetch_desc(&tm_ks);
      tma_prefetch_desc(&tm_vv);
      tma_prefetch_desc(&tm_vs);
      const int row0 = kh * p.n_ctx + c0;
      auto load = [&](const CUtensorMap* tv, const CUtensorMap* ts, int g, int item) {
        if (g >= nsub || *abort_flag) return;  // after a wait has given up nothing new is issued
        const int slot = item % NSLOT;
        uint8_t* raw = sgen + OFF_RAW + slot * ITEM_BYTES;
        int row = row0 + g * SUB;
        if (PAGED) {  // an item never straddles a page (64 | 256)
          const int pp = c0 + g * SUB;
          int pg = p.page_table[(size_t)seq * p.max_pages + pp / Q27B_PAGE];
          if (pg < 0 || pg >= p.n_pages) {  // never read outside the pool: flag it and read page 0
            atomicOr(p.status, ST_BAD_PAGE);
            pg = 0;
          }
          row = (pg * p.nkvh + kh) * Q27B_PAGE + pp % Q27B_PAGE;
        }
        mbar_wait(&bar[B_RAWEMPTY + slot], ((item / NSLOT) & 1) ^ 1, abort_flag, p.status);
        mbar_expect_tx(&bar[B_RAWFULL + slot], ITEM_BYTES);
        tma_load_2d(raw, tv, 0, row, &bar[B_RAWFULL + slot]);
        tma_load_2d(raw + SEG, tv, 128, row, &bar[B_RAWFULL + slot]);
        tma_load_2d(raw + I_SC, ts, 0, row, &bar[B_RAWFULL + slot]);
      };
      _Pragma("unroll 1") for (int g = 0; g < 4; g++) load(&tm_kv, &tm_ks, g, g);
      _Pragma("unroll 1") for (int j = 0; j < nt; j++) {
        load(&tm_vv, &tm_vs, 2 * j, v_item(j, 0));
        load(&tm_vv, &tm_vs, 2 * j + 1, v_item(j, 1));
        load(&tm_kv, &tm_ks, 2 * j + 4, k_item(j + 2, 0));
        load(&tm_kv, &tm_ks, 2 * j + 5, k_item(j + 2, 1));
      }
    }
  } else if (warp == QK_WARP) {
    // ================================================================ issuer of S^T = K Q^T
    if (lane == 0) {
      mbar_wait(&bar[B_QFULL], 0, abort_flag, p.status);
      _Pragma("unroll 1") for (int j = 0; j < nt && !*abort_flag; j++) {
        const int slot = j & 1;
        mbar_wait(&bar[B_SEMPTY + slot], ((j >> 1) & 1) ^ 1, abort_flag, p.status);
#pragma unroll
        for (int h = 0; h < 2; h++) {
          mbar_wait(&bar[B_KTFULL + h], j & 1, abort_flag, p.status);
          tc_fence_after();
#pragma unroll
          for (int k8 = 0; k8 < 8; k8++) {
            const int kk = h * 8 + k8;
            // A = K[128 positions][16 dims] in TMEM, B = Q^T[32 rows][16 dims]
            const uint64_t db = umma_desc_sw128(sbase + OFF_Q + (kk >> 2) * QSEG + (kk & 3) * 32, 16, 1024);
            tc_mma_f16_ts(tmem + TM_S + slot * 32, tmem + TM_K + kk * 8, db, IDESC_QK, kk > 0 ? 1u : 0u);
          }
          tc_commit(&bar[B_KTEMPTY + h]);
        }
        tc_commit(&bar[B_SFULL + slot]);
      }
    }
  } else {
    // ================================================================ issuer of O += P V
    if (lane == 0) {
      _Pragma("unroll 1") for (int j = 0; j < nt && !*abort_flag; j++) {
        const int ns = min(2, nsub - 2 * j);
        mbar_wait(&bar[B_PTFULL], j & 1, abort_flag, p.status);
        _Pragma("unroll 1") for (int s = 0; s < ns; s++) {
          mbar_wait(&bar[B_VFFULL + s], j & 1, abort_flag, p.status);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < SUB / 16; kk++) {
            // A = P[128 rows][16 positions] in TMEM, B = V[16 positions][256 dims], MN-major
            const uint64_t db = umma_desc_sw128(sbase + OFF_VF + s * VF_BYTES + kk * 2048, SEG, 1024);
            tc_mma_f16_ts(tmem + TM_O, tmem + TM_P + (s * 4 + kk) * 8, db, IDESC_PV, (j > 0 || s > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&bar[B_VFEMPTY + s]);
        }
        tc_commit(&bar[B_PTEMPTY]);
      }
      tc_commit(&bar[B_ODONE]);
    }
  }

  drain_after_abort(abort_flag);
  tc_fence_before();
  __syncthreads();
  if (warp == QK_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace

int launch_decode_tc(const CUtensorMap* kv, const CUtensorMap* ks, const CUtensorMap* vv, const CUtensorMap* vs,
                     const DecodeParams& p, bool paged, int nseq, cudaStream_t s) {
  static bool attr[64] = {};
  int dev;
  Q27B_CK(cudaGetDevice(&dev));
  if (!attr[dev]) {
    Q27B_CK(cudaFuncSetAttribute(decode_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
    Q27B_CK(cudaFuncSetAttribute(decode_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES));
    attr[dev] = true;
  }
  const dim3 grid(p.nch, p.nkvh, nseq);
  if (paged) Q27B_CK(launch_pdl(decode_tc_kernel<true>, grid, dim3(TC_THREADS), TC_SMEM_BYTES, s, *kv, *ks, *vv, *vs, p));
  else Q27B_CK(launch_pdl(decode_tc_kernel<false>, grid, dim3(TC_THREADS), TC_SMEM_BYTES, s, *kv, *ks, *vv, *vs, p));
  return Q27B_OK;
}

}  // namespace q27b
