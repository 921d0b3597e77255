// Causal flash-attention prefill over an f16 KV cache: Q K^T and P V both on tcgen05.mma kind::f16.
//
// The f16-QK variant of the reference (attn_prefill_kernel<PT, false>, src/attn.cu:338-528, used
// for f16 caches): Q * kq_scale rounded to f16, K and V as stored, S in f32, P -> f16, online
// softmax. Unlike the reference, O accumulates in f32 (in TMEM), so its max offset (P <= 1/8,
// src/attn.cu:323) is not needed; the reference max of a row moves only when the true max has
// grown by more than TAU. The 64-position K and V tiles that TMA brings from the cache are the
// operands of the tensor core as they land ([64-dim segment][position][128 B], 128-byte swizzle:
// K-major for K, read MN-major for V; ring of three stages each): no converter warps, no per-block
// scale arithmetic.
//
// One CTA = 128 query tokens of one query head (TMEM lane = token) x one split of the positions.
// Warps 0-7 softmax (two warpgroups, 32 columns of a tile each), warp 8 TMA producer, warp 9 issues
// the Q K^T MMAs (per tile 16 x (128x64x16) into one of two S buffers), warp 10 the P V MMAs
// (4 x (128x256x16) into O).
// TMEM: columns 0-255 O (f32), 256-383 two S buffers of 64 columns (f32), 384-511 the Q tile (f16
// pairs), the A operand of every Q K^T MMA (tcgen05.mma with A in tensor memory).
//
// Q8 = true: the same on a q8_0 cache, the reference's path with Q27_ATTN_I8=0
// (attn_prefill_kernel<PT, true>, src/attn.cu:338-528): K and V are dequantised to f16 (q * d rounded
// once, cvt_q8_16 src/attn.cu:59-76) on their way to the tensor core. TMA brings the int8 tiles and
// their scales into raw stages, warps 11-14 turn K and warps 15-18 turn V into the f16 operand
// layout above (two f16 buffers and two raw stages per operand).
#include "combine.h"
#include "common.cuh"
#include "prefill_f16.h"

#include <mutex>

#include <algorithm>
#include <cstdlib>

namespace q27b {
namespace {

constexpr int QT = 128;          // query tokens per CTA
constexpr int PT = 64;           // positions per tile
constexpr float TAU = 5.0f;
constexpr int SEGK = PT * 128;   // one 64-dim segment of a K or V tile: [64 positions][128 B]
constexpr int KV_BYTES = 4 * SEGK;          // 32 KB
constexpr int P_BYTES = QT * 128;           // f16 P: [128][64 positions]
constexpr int RAW_BYTES = 2 * PT * 128 + PT * 16;  // q8_0 tile: two 128-dim int8 segments [64][128 B], then [64][8] f16 scales
enum { B_QFULL = 0, B_KFULL = 1, B_KEMPTY = 4, B_VFULL = 7, B_VEMPTY = 10, B_SFULL = 13, B_SEMPTY = 15, B_PFULL = 17, B_PEMPTY = 18, B_ODONE = 19,
       B_RKFULL = 20, B_RKEMPTY = 22, B_RVFULL = 24, B_RVEMPTY = 26, NBAR = 28 };
// Shared memory. f16 cache: three K and three V stages, filled by TMA. q8_0 cache: two f16 K and two
// f16 V buffers, filled by the converter warps from two raw stages each. (The Q tile is in TMEM.)
template <bool Q8, int NWG>
struct Lay {
  static constexpr int NKF = Q8 ? 2 : 3;                   // f16 K buffers, and as many f16 V buffers
  static constexpr int NSW = 4 * NWG;                      // softmax warps: NWG threads per query row
  // The P V MMAs have an issuing thread of their own: measured +10 % on an f16 cache and +11-15 % on
  // a q8_0 cache (with one f16 buffer per operand instead of two it had lost 11 % there).
  static constexpr bool SPLIT_ISSUE = true;
  static constexpr int TMA_WARP = NSW, MMA_WARP = NSW + 1, PV_WARP = SPLIT_ISSUE ? NSW + 2 : -1;
  static constexpr int KCONV_WARP0 = NSW + 2 + SPLIT_ISSUE, VCONV_WARP0 = KCONV_WARP0 + 4;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + NKF * KV_BYTES;
  static constexpr int OFF_P = OFF_V + NKF * KV_BYTES;     // one buffer
  static constexpr int OFF_RAW = OFF_P + P_BYTES;          // q8_0: K stage 0, 1, V stage 0, 1
  static constexpr int OFF_XCH = OFF_RAW + (Q8 ? 4 * RAW_BYTES : 0);  // [tile parity][NWG][128] f32
  static constexpr int OFF_BAR = OFF_XCH + 2 * NWG * QT * 4;
  static constexpr int OFF_MISC = OFF_BAR + NBAR * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;
  static constexpr int THREADS = (NSW + 2 + SPLIT_ISSUE + (Q8 ? 8 : 0)) * 32;
  static_assert(OFF_K % 1024 == 0 && OFF_V % 1024 == 0 && OFF_P % 1024 == 0 && OFF_RAW % 1024 == 0 && RAW_BYTES % 1024 == 0,
                "swizzled tiles need 1024-byte alignment");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");
};

constexpr int N_CONV_WARPS = 4;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_O = 0, TM_S = 256, TM_Q = 384;  // O f32 256 columns, S 2 x 64 f32, Q 128 columns of f16 pairs
constexpr uint32_t IDESC_QK = umma_idesc(1, 0, 0, 0, 0, QT, PT);   // f32 += f16 * f16, both K-major, M128 N64
constexpr uint32_t IDESC_PV = umma_idesc(1, 0, 0, 0, 1, QT, AD);   // B (V) MN-major, M128 N256

struct F16Params {
  const float* qn;   // [M][nqh][256]
  const float* qg;   // [M][nqh][512]
  float* o;          // [M][nqh][256]
  float* part;       // [nsplit][Ms][nqh][258], Ms = min(M, 128 ts): the tokens whose positions are split
  const int* pos0;
  int* status;
  int M, nqh, nkvh, n_ctx;
  int ts, nsplit;    // query tiles [0, ts) are split nsplit ways over their positions, the others are not
  float kq_scale;
};

// the NWG threads of a query row sit in warp q of every softmax warpgroup
template <int NWG>
__device__ __forceinline__ void row_sync(int q) { asm volatile("bar.sync %0, %1;" ::"r"(1 + q), "n"(32 * NWG) : "memory"); }

// Rare, and kept out of line: inlined, its 32 registers of payload would sit on the loop's state.
__device__ __noinline__ void rescale_o_f16(uint32_t taddr, float f, int chunks) {
#pragma unroll 1
  for (int c = 0; c < chunks; c++) {
    uint32_t v[32];
    tmem_ld32(taddr + c * 32, v);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
    tmem_st32(taddr + c * 32, v);
  }
}

// One tile of a q8_0 cache, raw stage -> f16 operand buffer. 128 threads; item = (row, 16-dim chunk);
// eight neighbouring lanes take 4 chunks of rows rho and rho ^ 5, which keeps both the swizzled
// 16-byte loads and the swizzled 16-byte stores free of bank conflicts. Thread ct owns the same chunk
// of rows row0, row0 + 8, .., row0 + 56: rows 8 apart share their swizzle phase, so every address is
// a per-thread base (ConvAddr, computed once per kernel) plus a constant. Rows >= zero_from are
// cleared (rows past the sequence may hold anything: P is 0 there, V must be too).
struct ConvAddr {
  int row0;       // first row of this thread
  uint32_t src;   // byte offset of its 16 int8 values of row0 in the raw stage
  uint32_t sc;    // ... of their f16 scale
  uint32_t dst;   // ... of the first of its two 16-byte chunks in the f16 buffer
};
__device__ __forceinline__ ConvAddr conv_addr(int ct) {
  ConvAddr a;
  a.row0 = (2 * (ct >> 5)) ^ (5 * ((ct >> 2) & 1));
  const int c16 = (ct & 3) + 4 * ((ct >> 3) & 3);
  a.src = (c16 >> 3) * (PT * 128) + swz128(a.row0, c16 & 7);
  a.sc = 2 * PT * 128 + a.row0 * 16 + (c16 >> 1) * 2;
  a.dst = (c16 >> 2) * SEGK + swz128(a.row0, 2 * (c16 & 3));
  return a;
}
__device__ __forceinline__ void convert_q8_tile(const uint8_t* raw, uint8_t* dst_tile, const ConvAddr& a, int zero_from) {
#pragma unroll 1
  for (int k0 = 0; k0 < 8; k0 += 4) {
    // loads of four items first: a shared-memory load is never moved above an earlier store
    uint4 x[4];
    __half d[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      x[k] = *(const uint4*)(raw + a.src + (k0 + k) * 1024);
      d[k] = *(const __half*)(raw + a.sc + (k0 + k) * 128);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const __half2 dd = __half2half2(d[k]);
      const uint32_t xw[4] = {x[k].x ^ 0x80808080u, x[k].y ^ 0x80808080u, x[k].z ^ 0x80808080u, x[k].w ^ 0x80808080u};
      uint32_t o[8];
#pragma unroll
      for (int w = 0; w < 4; w++) {
        o[2 * w] = dq_pair(__byte_perm(xw[w], 0x64646464u, 0x4140), dd);
        o[2 * w + 1] = dq_pair(__byte_perm(xw[w], 0x64646464u, 0x4342), dd);
      }
      if (a.row0 + 8 * (k0 + k) >= zero_from) {
#pragma unroll
        for (int w = 0; w < 8; w++) o[w] = 0;
      }
      uint8_t* dst = dst_tile + (k0 + k) * 1024;
      *(uint4*)(dst + a.dst) = make_uint4(o[0], o[1], o[2], o[3]);
      *(uint4*)(dst + (a.dst ^ 16u)) = make_uint4(o[4], o[5], o[6], o[7]);
    }
  }
}

// tm_k, tm_v: f16 cache rows (f16 cache) or the int8 values (q8_0 cache); tm_ks, tm_vs: the q8_0 scales.
template <bool Q8, int NWG>
__global__ void __launch_bounds__(Lay<Q8, NWG>::THREADS, 1)
prefill_f16_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_ks, const __grid_constant__ CUtensorMap tm_vs, const F16Params p) {
  using LY = Lay<Q8, NWG>;
  constexpr int N_SOFTMAX_WARPS = LY::NSW, TMA_WARP = LY::TMA_WARP, MMA_WARP = LY::MMA_WARP, PV_WARP = LY::PV_WARP,
                KCONV_WARP0 = LY::KCONV_WARP0, VCONV_WARP0 = LY::VCONV_WARP0;
  (void)VCONV_WARP0;
  constexpr int CW = PT / NWG;    // columns (positions) of a tile per softmax thread
  constexpr int OW = AD / NWG;    // columns of O per softmax thread (rescale, epilogue)
  constexpr int NKF = LY::NKF, OFF_K = LY::OFF_K, OFF_V = LY::OFF_V, OFF_P = LY::OFF_P, OFF_RAW = LY::OFF_RAW,
                OFF_XCH = LY::OFF_XCH, OFF_BAR = LY::OFF_BAR, OFF_MISC = LY::OFF_MISC;
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  uint64_t* bar = (uint64_t*)(sgen + OFF_BAR);
  uint32_t* tmem_slot = (uint32_t*)(sgen + OFF_MISC);
  volatile int* abort_flag = (volatile int*)(sgen + OFF_MISC + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // CTA order: the unsplit CTAs (tiles >= ts) first, then the pieces of the split tiles, split index
  // slowest; within each class head by head, the query tiles with the most positions first
  // (src/attn.cu:567)
  int L = (int)blockIdx.x, z = 0, nsplit = 1, ntl = (p.M + QT - 1) / QT - p.ts, tile_base = p.ts;
  if (L >= ntl * p.nqh) {
    L -= ntl * p.nqh;
    ntl = p.ts;
    tile_base = 0;
    nsplit = p.nsplit;
    z = L / (ntl * p.nqh);
    L -= z * ntl * p.nqh;
  }
  const int h = L / ntl, kh = h / GQA;
  const int t0 = (tile_base + ntl - 1 - L % ntl) * QT;
  const int Ms = min(p.M, p.ts * QT);
  const int pos0 = *p.pos0;
  const int n_end = min(pos0 + min(t0 + QT, p.M), p.n_ctx);
  const int ntot = (n_end + PT - 1) / PT;
  const int per = (ntot + nsplit - 1) / nsplit;
  const int it0 = min(ntot, z * per), it1 = min(ntot, it0 + per);
  const int nt = it1 - it0;

  if (nt <= 0) {  // nothing in this split: neutral partials
    if (nsplit > 1 && tid < QT && t0 + tid < p.M) {
      float* po = p.part + (((size_t)z * Ms + t0 + tid) * p.nqh + h) * PROW;
      po[0] = M_INIT;
      po[1] = 0.f;
      for (int d = 0; d < AD; d++) po[2 + d] = 0.f;
    }
    return;
  }

  if (tid == 0) {
    mbar_init(&bar[B_QFULL], N_SOFTMAX_WARPS);
    for (int s = 0; s < 3; s++) {
      mbar_init(&bar[B_KFULL + s], Q8 ? N_CONV_WARPS : 1);  // q8_0: the converter warps fill the buffers
      mbar_init(&bar[B_KEMPTY + s], 1);
      mbar_init(&bar[B_VFULL + s], Q8 ? N_CONV_WARPS : 1);
      mbar_init(&bar[B_VEMPTY + s], 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(&bar[B_SFULL + s], 1);
      mbar_init(&bar[B_SEMPTY + s], N_SOFTMAX_WARPS);
      mbar_init(&bar[B_RKFULL + s], 1);
      mbar_init(&bar[B_RKEMPTY + s], N_CONV_WARPS);
      mbar_init(&bar[B_RVFULL + s], 1);
      mbar_init(&bar[B_RVEMPTY + s], N_CONV_WARPS);
    }
    mbar_init(&bar[B_PFULL], N_SOFTMAX_WARPS);
    mbar_init(&bar[B_PEMPTY], 1);
    mbar_init(&bar[B_ODONE], 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < N_SOFTMAX_WARPS) {
    // ================================================================ softmax warps
    const int wg = warp >> 2, q = warp & 3;
    const int r = q * 32 + lane;       // query row = TMEM lane
    const int t = t0 + r;
    const bool live = t < p.M;
    float* xch = (float*)(sgen + OFF_XCH);
    const uint32_t tlane = tmem + ((uint32_t)(q * 32) << 16);
    {
      // Q tile -> tensor memory, the A operand of every Q K^T MMA of this CTA (lane = row, column c =
      // dims 2c, 2c+1 as f16, even dim in the low half): it is read from there 16 times per tile
      // without touching shared memory. This thread writes dims OW wg .. OW wg + OW - 1 of its row,
      // scaled and rounded to f16; rows past M are zero.
      const float* src = live ? p.qn + ((size_t)t * p.nqh + h) * AD + OW * wg : nullptr;
#pragma unroll 1
      for (int c = 0; c < OW / 64; c++) {
        uint32_t w[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float4 a = src ? *(const float4*)(src + c * 64 + 2 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
          w[i] = pack_h2(a.x * p.kq_scale, a.y * p.kq_scale);
          w[i + 1] = pack_h2(a.z * p.kq_scale, a.w * p.kq_scale);
        }
        tmem_st32(tlane + TM_Q + wg * (OW / 2) + c * 32, w);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_QFULL]);
    }

    const int limit = pos0 + t + 1;    // positions < limit are visible
    const int col0 = wg * CW;          // this thread's positions of a tile
    float m_run = M_INIT, m_ref = M_INIT;
    uint64_t l2 = pack2(0.f, 0.f);
    const uint64_t log2e2 = pack2(LOG2E, LOG2E);

#pragma unroll 1
    for (int j = 0; j < nt; j++) {
      const int slot = j & 1;
      const int p_tile = (it0 + j) * PT;
      mbar_wait(&bar[B_SFULL + slot], (j >> 1) & 1, abort_flag, p.status);
      tc_fence_after();
      float s[CW];
      {
        uint32_t v[CW];
        tmem_ld(tlane + TM_S + slot * PT + col0, v);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < CW; i++) s[i] = __uint_as_float(v[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_SEMPTY + slot]);  // the buffer is in registers: it can be overwritten

      // causal mask (only tiles that reach past the first row's limit need it) and this thread's max
      if (p_tile + PT > pos0 + t0 + 1) {
#pragma unroll
        for (int i = 0; i < CW; i++)
          if (p_tile + col0 + i >= limit) s[i] = -INFINITY;
      }
      float mq[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < CW; i += 4) {
        mq[0] = fmaxf(mq[0], s[i]);
        mq[1] = fmaxf(mq[1], s[i + 1]);
        mq[2] = fmaxf(mq[2], s[i + 2]);
        mq[3] = fmaxf(mq[3], s[i + 3]);
      }
      float mt = fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3]));
      // row maximum over the NWG threads of the row; the buffer alternates with the tile
      xch[(slot * NWG + wg) * QT + r] = mt;
      row_sync<NWG>(q);
#pragma unroll
      for (int o = 1; o < NWG; o++) mt = fmaxf(mt, xch[(slot * NWG + ((wg + o) % NWG)) * QT + r]);
      m_run = fmaxf(m_run, mt);

      // Move the reference max when the true max has run away from it (and on the first tile). The
      // threads of a row hold the same m_run and m_ref, so their warps take the same branch.
      const bool want = m_run > m_ref + TAU;
      if (__any_sync(0xffffffffu, want)) {
        const float f = ex2((m_ref - m_run) * LOG2E);  // 0 on the first move (m_ref = -1e30)
        m_ref = m_run;
        l2 = mul2(l2, pack2(f, f));
        if (j > 0) {
          // O holds the sum of tiles < j once the P V of tile j-1 has completed
          mbar_wait(&bar[B_PEMPTY], (j - 1) & 1, abort_flag, p.status);
          tc_fence_after();
          rescale_o_f16(tlane + TM_O + wg * OW, f, OW / 32);
          tc_wait_st();
          tc_fence_before();
        }
      }

      // P = exp(s - m_ref): f32 row sum, f16 for the P V MMA (16-byte chunks CW/8 wg .. of the row)
      mbar_wait(&bar[B_PEMPTY], (j & 1) ^ 1, abort_flag, p.status);  // P V of tile j-1 has read the buffer
      uint8_t* sP = sgen + OFF_P;
      const float nmb = -m_ref * LOG2E;
      const uint64_t nmb2 = pack2(nmb, nmb);
#pragma unroll
      for (int c = 0; c < CW / 8; c++) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          float a0, a1;
          unpack2(fma2(pack2(s[c * 8 + 2 * k], s[c * 8 + 2 * k + 1]), log2e2, nmb2), a0, a1);
          const float e0 = ex2(a0), e1 = ex2(a1);
          l2 = add2(l2, pack2(e0, e1));
          w[k] = pack_h2(e0, e1);
        }
        *(uint4*)(sP + swz128(r, CW / 8 * wg + c)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (!Q8 && p_tile + PT > n_end) {
        // The last tile reaches past the sequence: those cache rows hold whatever was there before
        // (possibly NaN or Inf, and 0 * NaN = NaN in the P V product), so the V rows past the end are
        // cleared in shared memory. Thread = (segment, position); a row of a segment is 128 bytes,
        // and the swizzle only permutes within it.
        const int vb = j % NKF;
        mbar_wait(&bar[B_VFULL + vb], (j / NKF) & 1, abort_flag, p.status);
        for (int u = tid; u < 4 * PT; u += 32 * N_SOFTMAX_WARPS) {
          const int sg = u >> 6, row = u & 63;
          if (p_tile + row >= n_end) {
            uint4* vrow = (uint4*)(sgen + OFF_V + vb * KV_BYTES + sg * SEGK + row * 128);
#pragma unroll
            for (int c = 0; c < 8; c++) vrow[c] = make_uint4(0, 0, 0, 0);
          }
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_PFULL]);
    }

    // ---- epilogue: O / l * sigmoid(gate), or the unnormalised partial of this split
    float la, lb;
    unpack2(l2, la, lb);
    float l = la + lb;
    xch[((nt & 1) * NWG + wg) * QT + r] = l;
    row_sync<NWG>(q);
#pragma unroll
    for (int o = 1; o < NWG; o++) l += xch[((nt & 1) * NWG + ((wg + o) % NWG)) * QT + r];
    mbar_wait(&bar[B_ODONE], 0, abort_flag, p.status);
    tc_fence_after();
    const float inv_l = 1.0f / l;
    float* po = nsplit > 1 ? p.part + (((size_t)z * Ms + t) * p.nqh + h) * PROW : nullptr;
    if (live && po && wg == 0) {
      po[0] = m_ref;
      po[1] = l;
    }
#pragma unroll 1
    for (int c = 0; c < OW / 32; c++) {
      const int d0 = wg * OW + c * 32;
      uint32_t v[32];
      tmem_ld32(tlane + TM_O + d0, v);
      tc_wait_ld();
      if (!live) continue;
      if (po) {
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          *(float2*)(po + 2 + d0 + i) = make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      } else {
        const float* gt = p.qg + ((size_t)t * p.nqh + h) * 512 + 256 + d0;
        float* dst = p.o + ((size_t)t * p.nqh + h) * AD + d0;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 gg = *(const float4*)(gt + i);
          float4 y;
          y.x = (__uint_as_float(v[i]) * inv_l) * (1.0f / (1.0f + __expf(-gg.x)));
          y.y = (__uint_as_float(v[i + 1]) * inv_l) * (1.0f / (1.0f + __expf(-gg.y)));
          y.z = (__uint_as_float(v[i + 2]) * inv_l) * (1.0f / (1.0f + __expf(-gg.z)));
          y.w = (__uint_as_float(v[i + 3]) * inv_l) * (1.0f / (1.0f + __expf(-gg.w)));
          *(float4*)(dst + i) = y;
        }
      }
    }
    tc_fence_before();
  } else if (warp == TMA_WARP) {
    // ================================================================ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      if (Q8) {
        tma_prefetch_desc(&tm_ks);
        tma_prefetch_desc(&tm_vs);
      }
#pragma unroll 1
      for (int j = 0; j < nt; j++) {
        const int row = kh * p.n_ctx + (it0 + j) * PT;
        if constexpr (Q8) {
          const int st = j & 1, ph = (j >> 1) & 1;  // raw stages
          uint8_t* kr = sgen + OFF_RAW + st * RAW_BYTES;
          uint8_t* vr = sgen + OFF_RAW + (2 + st) * RAW_BYTES;
          mbar_wait(&bar[B_RKEMPTY + st], ph ^ 1, abort_flag, p.status);
          mbar_expect_tx(&bar[B_RKFULL + st], RAW_BYTES);
          tma_load_2d(kr, &tm_k, 0, row, &bar[B_RKFULL + st]);
          tma_load_2d(kr + PT * 128, &tm_k, 128, row, &bar[B_RKFULL + st]);
          tma_load_2d(kr + 2 * PT * 128, &tm_ks, 0, row, &bar[B_RKFULL + st]);
          mbar_wait(&bar[B_RVEMPTY + st], ph ^ 1, abort_flag, p.status);
          mbar_expect_tx(&bar[B_RVFULL + st], RAW_BYTES);
          tma_load_2d(vr, &tm_v, 0, row, &bar[B_RVFULL + st]);
          tma_load_2d(vr + PT * 128, &tm_v, 128, row, &bar[B_RVFULL + st]);
          tma_load_2d(vr + 2 * PT * 128, &tm_vs, 0, row, &bar[B_RVFULL + st]);
        } else {
          const int st = j % NKF, ph = (j / NKF) & 1;
          uint8_t* ks = sgen + OFF_K + st * KV_BYTES;
          uint8_t* vs = sgen + OFF_V + st * KV_BYTES;
          mbar_wait(&bar[B_KEMPTY + st], ph ^ 1, abort_flag, p.status);
          mbar_expect_tx(&bar[B_KFULL + st], KV_BYTES);
#pragma unroll
          for (int sg = 0; sg < 4; sg++) tma_load_2d(ks + sg * SEGK, &tm_k, sg * 128, row, &bar[B_KFULL + st]);
          mbar_wait(&bar[B_VEMPTY + st], ph ^ 1, abort_flag, p.status);
          mbar_expect_tx(&bar[B_VFULL + st], KV_BYTES);
#pragma unroll
          for (int sg = 0; sg < 4; sg++) tma_load_2d(vs + sg * SEGK, &tm_v, sg * 128, row, &bar[B_VFULL + st]);
        }
      }
    }
  } else if (Q8 && warp >= KCONV_WARP0) {
    // ================================================================ converter warps (q8_0 cache)
    const bool is_v = warp >= VCONV_WARP0;
    const int ct = tid - (is_v ? VCONV_WARP0 : KCONV_WARP0) * 32;
    const int b_rfull = is_v ? B_RVFULL : B_RKFULL, b_rempty = is_v ? B_RVEMPTY : B_RKEMPTY;
    const int b_full = is_v ? B_VFULL : B_KFULL, b_empty = is_v ? B_VEMPTY : B_KEMPTY;
    const ConvAddr ca = conv_addr(ct);
#pragma unroll 1
    for (int j = 0; j < nt; j++) {
      const int st = j & 1, fb = j % NKF;
      mbar_wait(&bar[b_rfull + st], (j >> 1) & 1, abort_flag, p.status);
      mbar_wait(&bar[b_empty + fb], ((j / NKF) & 1) ^ 1, abort_flag, p.status);  // the MMAs of tile j-NKF have read the buffer
      convert_q8_tile(sgen + OFF_RAW + ((is_v ? 2 : 0) + st) * RAW_BYTES, sgen + (is_v ? OFF_V : OFF_K) + fb * KV_BYTES, ca,
                      is_v ? n_end - (it0 + j) * PT : PT);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bar[b_full + fb]);
        mbar_arrive(&bar[b_rempty + st]);
      }
    }
  } else if (warp == MMA_WARP || warp == PV_WARP) {
    // ================================================================ MMA issuers
    // Operand buffer and phase of tile j: ring of NKF TMA stages (f16 cache) or converted buffers (q8_0).
    auto issue_pv = [&](int jj) {
      const int st = jj % NKF, ph = (jj / NKF) & 1;
      mbar_wait(&bar[B_PFULL], jj & 1, abort_flag, p.status);
      mbar_wait(&bar[B_VFULL + st], ph, abort_flag, p.status);
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < PT / 16; kk++) {
        const uint64_t da = umma_desc_sw128(sbase + OFF_P + kk * 32, 16, 1024);
        const uint64_t db = umma_desc_sw128(sbase + OFF_V + st * KV_BYTES + kk * 2048, SEGK, 1024);
        tc_mma_f16(tmem + TM_O, da, db, IDESC_PV, (jj > 0 || kk > 0) ? 1u : 0u);
      }
      tc_commit(&bar[B_PEMPTY]);
      tc_commit(&bar[B_VEMPTY + st]);
    };
    if (LY::SPLIT_ISSUE && warp == PV_WARP) {
      // P V from a thread of its own: a single thread issues the 128x64x16 MMAs of Q K^T at about
      // half the rate the tensor pipe could run them, and the P V MMAs of the previous tile fill the gaps
      if (lane == 0) {
#pragma unroll 1
        for (int jj = 0; jj < nt; jj++) issue_pv(jj);
        tc_commit(&bar[B_ODONE]);
      }
    } else if (lane == 0) {
      mbar_wait(&bar[B_QFULL], 0, abort_flag, p.status);
      tc_fence_after();
#pragma unroll 1
      for (int j = 0; j < nt; j++) {
        const int ss = j & 1, sph = (j >> 1) & 1;                         // S buffer
        const int st = j % NKF, ph = (j / NKF) & 1;                       // K buffer
        mbar_wait(&bar[B_KFULL + st], ph, abort_flag, p.status);
        mbar_wait(&bar[B_SEMPTY + ss], sph ^ 1, abort_flag, p.status);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < AD / 16; kk++) {
          const uint64_t db = umma_desc_sw128(sbase + OFF_K + st * KV_BYTES + (kk >> 2) * SEGK + (kk & 3) * 32, 16, 1024);
          tc_mma_f16_ts(tmem + TM_S + ss * PT, tmem + TM_Q + kk * 8, db, IDESC_QK, kk > 0 ? 1u : 0u);
        }
        tc_commit(&bar[B_SFULL + ss]);
        tc_commit(&bar[B_KEMPTY + st]);
        if (!LY::SPLIT_ISSUE && j >= 1) issue_pv(j - 1);
      }
      if (!LY::SPLIT_ISSUE) {
        issue_pv(nt - 1);
        tc_commit(&bar[B_ODONE]);
      }
    }
  }

  drain_after_abort(abort_flag);
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace

int launch_prefill_f16(DeviceCtx* ctx, const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                       int8_t* xq, float* xd, const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx, bool q8,
                       int depth_hint, cudaStream_t s) {
  static bool attr[64] = {};
  static std::mutex attr_mu;
  std::lock_guard<std::mutex> attr_lock(attr_mu);
  if (!attr[ctx->dev]) {
    Q27B_CK(cudaFuncSetAttribute(prefill_f16_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay<false, 2>::SMEM_BYTES));
    Q27B_CK(cudaFuncSetAttribute(prefill_f16_kernel<false, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay<false, 4>::SMEM_BYTES));
    Q27B_CK(cudaFuncSetAttribute(prefill_f16_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay<true, 2>::SMEM_BYTES));
    attr[ctx->dev] = true;
  }
  static const int nwg_f16 = [] { const char* e = getenv("Q27B_PF16_NWG"); return e && e[0] == '4' ? 4 : 2; }();
  const int tiles = (M + QT - 1) / QT;
  // splits over the positions as for the int8 kernel; the q8_1 output is written by the merge kernel,
  // so it needs every tile on the split path (at least one merge)
  SplitPlan sp = plan_prefill_split(tiles, nqh, ctx->n_sm, M, depth_hint, xq != nullptr);
  float* part;  // the fixed prefill workspace; the plan is cut to what it holds
  if (int rc = fit_prefill_split(ctx, &sp.ts, &sp.ns, M, nqh, xq != nullptr, &part)) return rc;
  const int nsplit = sp.ns, Ms = std::min(M, sp.ts * QT);
  CUtensorMap tkm, tvm, tksm, tvsm;
  const uint64_t rows = (uint64_t)nkvh * n_ctx;
  if (q8) {
    if (int rc = q8_tmaps(kcache, rows, &tkm, &tksm)) return rc;
    if (int rc = q8_tmaps(vcache, rows, &tvm, &tvsm)) return rc;
  } else {
    // rows of 512 bytes (256 halves), fetched as 128-byte wide, 64-row boxes with the 128-byte swizzle
    if (int rc = cached_tmap_2d(&tkm, kcache, rows, 2 * AD, 2 * AD, 128, PT, true)) return rc;
    if (int rc = cached_tmap_2d(&tvm, vcache, rows, 2 * AD, 2 * AD, 128, PT, true)) return rc;
    tksm = tkm;  // not read
    tvsm = tvm;
  }
  const CUtensorMap *tk = &tkm, *tv = &tvm, *tks = &tksm, *tvs = &tvsm;
  F16Params p = {};
  p.qn = qn; p.qg = qg; p.o = o; p.part = nsplit > 1 ? part : nullptr; p.pos0 = pos0; p.status = ctx->status;
  p.M = M; p.nqh = nqh; p.nkvh = nkvh; p.n_ctx = n_ctx; p.ts = sp.ts; p.nsplit = nsplit; p.kq_scale = kq_scale;
  const int grid = (tiles - sp.ts) * nqh + sp.ts * nqh * nsplit;
  if (q8)
    prefill_f16_kernel<true, 2><<<grid, Lay<true, 2>::THREADS, Lay<true, 2>::SMEM_BYTES, s>>>(*tk, *tv, *tks, *tvs, p);
  else if (nwg_f16 == 4)
    prefill_f16_kernel<false, 4><<<grid, Lay<false, 4>::THREADS, Lay<false, 4>::SMEM_BYTES, s>>>(*tk, *tv, *tks, *tvs, p);
  else
    prefill_f16_kernel<false, 2><<<grid, Lay<false, 2>::THREADS, Lay<false, 2>::SMEM_BYTES, s>>>(*tk, *tv, *tks, *tvs, p);
  Q27B_CK(cudaGetLastError());
  if (nsplit > 1) {  // the split tokens are rows [0, Ms * nqh) of every array
    MergeParams mp = {};
    mp.part = part; mp.nparts = nsplit; mp.part_stride = (int64_t)Ms * nqh * PROW; mp.rows = (int64_t)Ms * nqh;
    mp.qg = qg; mp.o = o; mp.xq = xq; mp.xd = xd;
    return launch_merge(mp, false, s);
  }
  return Q27B_OK;
}

}  // namespace q27b
