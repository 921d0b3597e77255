// Causal flash-attention prefill over a q8_0 KV cache with int8 Q K^T on the 5th-generation
// tensor cores (tcgen05.mma kind::i8 into TMEM) and P V on kind::f16.
//
// Replaces attn_prefill_i8_kernel + the host wrapper attn_prefill of the reference
// (src/attn.cu:557-801, 920-974) with the same arithmetic definition: Q * kq_scale rounded to
// int8 with one f32 scale per 32 dims, K = the cache bytes as stored, one exact int32 dot product
// per 32-dim block, s = sum_b (dq[b] * dk[p][b]) * float(I_b) in block order, online softmax,
// P -> f16, V -> f16(int8 * f16 scale). Unlike the reference, O accumulates in f32 (in TMEM), so
// no max offset is needed; the reference max of a row is only moved when its true max has grown
// by more than TAU, which keeps P <= e^TAU and makes the O rescale rare.
//
// One CTA = 128 query tokens of one query head (TMEM lane = token) x one split of the positions,
// walking 64-position tiles. Roles (14 warps):
//   warps 0-7   softmax, two warpgroups: both own the 128 rows (warp w and w+4 share TMEM lanes
//               32(w%4)..), warpgroup 0 takes positions 0-31 of a tile, warpgroup 1 positions
//               32-63. Each thread reads its half of the per-block int32 accumulators from TMEM,
//               applies the block scales with packed f32x2 arithmetic, exchanges the row maximum
//               with its partner thread, writes its half of P (f16) into shared memory in the
//               tensor core's K-major 128B-swizzled layout, rescales its half of O when the
//               reference max moves, and writes its half of the output columns.
//   warps 8-11  converter: V tile int8 -> f16 into the MN-major 128B-swizzled layout that the P V
//               MMA reads directly (no transpose), and the K scales f16 -> f32 table.
//   warp 12     TMA producer (one lane): K and V tiles, double buffered.
//   warp 13     MMA issuer (one lane): per tile 8 x (128x64x32 int8) into a 4-slot ring of TMEM
//               accumulators, then 4 x (128x256x16 f16) into the O accumulator; owns TMEM.
// TMEM: columns 0-255 O (f32), 256-511 four S slots of 64 columns (s32).
#include "combine.h"
#include "common.cuh"
#include "prefill_f16.h"

#include <algorithm>
#include <atomic>

namespace q27b {
namespace {

constexpr int QT = 128;          // query tokens per CTA
constexpr int PT = 64;           // positions per tile
constexpr float TAU = 5.0f;      // the reference max moves only when the true max exceeds it by this much

// shared memory map (offsets from a 1024-byte aligned base)
constexpr int SQ_BYTES = 2 * QT * 128;              // int8 Q: two K-halves of [128][128 B]
constexpr int KST_BYTES = 2 * PT * 128 + PT * 16;   // one K (or V) stage: values + scales
constexpr int VF_BYTES = 4 * PT * 128;              // f16 V: [4 dim chunks][64 positions][128 B]
constexpr int P_BYTES = QT * 128;                   // f16 P: [128][64 positions]
constexpr int DKF_BYTES = 8 * PT * 4;               // f32 K scales [8 blocks][64]
constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + SQ_BYTES;             // 2 stages (each padded to 18432 = 18 KB)
constexpr int KST_PAD = 18432;
constexpr int OFF_V = OFF_K + 2 * KST_PAD;
constexpr int OFF_VF = OFF_V + 2 * KST_PAD;
constexpr int OFF_P = OFF_VF + 2 * VF_BYTES;
constexpr int OFF_DKF = OFF_P + 2 * P_BYTES;
constexpr int OFF_DQ = OFF_DKF + 2 * DKF_BYTES;     // f32 Q scales [8 blocks][128 rows] (a warp reads one block of 32 rows: no bank conflict)
constexpr int OFF_XCH = OFF_DQ + QT * 8 * 4;        // row exchange between the two softmax warpgroups [tile parity][2][128] f32
constexpr int OFF_BAR = OFF_XCH + 2 * 4 * QT * 4;   // room for four warpgroups
constexpr int NBAR = 32;
constexpr int OFF_MISC = OFF_BAR + NBAR * 8;        // tmem base address, abort flag
constexpr int PF_SMEM_USED = OFF_MISC + 16;
constexpr int PF_SMEM_BYTES = PF_SMEM_USED + 1024;
static_assert(KST_BYTES <= KST_PAD && KST_PAD % 1024 == 0, "stage padding");
static_assert(OFF_VF % 1024 == 0 && OFF_P % 1024 == 0 && OFF_K % 1024 == 0, "swizzled tiles need 1024-byte alignment");
static_assert(PF_SMEM_BYTES <= 232448, "shared memory budget of one CTA");

// mbarrier indices
enum {
  B_QFULL = 0,
  B_KFULL = 1,    // [2]
  B_KEMPTY = 3,   // [2]
  B_VFULL = 5,    // [2]
  B_VEMPTY = 7,   // [2]
  B_VFFULL = 9,   // [2]
  B_VFEMPTY = 11, // [2]
  B_DKEMPTY = 13, // [2]
  B_SFULL = 15,   // [4]
  B_SEMPTY = 19,  // [4]
  B_PFULL = 23,   // [2]
  B_PEMPTY = 25,  // [2]
  B_ODONE = 27,
};

#ifndef Q27B_PF_NWG
#define Q27B_PF_NWG 2
#endif
constexpr int NWG = Q27B_PF_NWG;               // softmax warpgroups: each takes PT / NWG columns of a tile
constexpr int WCOLS = PT / NWG;                // columns per softmax thread
constexpr int OCOLS = AD / NWG;                // columns of O per softmax thread (rescale, epilogue)
constexpr int N_SOFTMAX_WARPS = 4 * NWG;
constexpr int N_CONV_WARPS = 4;   // measured: 2 converter warps (and 162 registers for the softmax warps) lose 8 %
constexpr int N_CONV_THREADS = N_CONV_WARPS * 32;
constexpr int CONV_WARP0 = N_SOFTMAX_WARPS, TMA_WARP = CONV_WARP0 + N_CONV_WARPS, MMA_WARP = TMA_WARP + 1;
constexpr int PF_THREADS = (MMA_WARP + 1) * 32;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t TM_O = 0, TM_S = 256;
constexpr uint32_t IDESC_QK = umma_idesc(2, 1, 1, 0, 0, QT, PT);    // s32 += s8 * s8, both K-major, M128 N64
constexpr uint32_t IDESC_PV = umma_idesc(1, 0, 0, 0, 1, QT, AD);    // f32 += f16 * f16, B MN-major, M128 N256

struct PrefillParams {
  const float* qn;   // [M][nqh][256]
  const float* qg;   // [M][nqh][512]
  float* o;          // [M][nqh][256]
  float* part;       // [nsplit][Ms][nqh][258], Ms = min(M, 128 ts): the tokens whose positions are split
  const int* pos0;
  int* status;
  int M, nqh, nkvh, n_ctx;
  int ts, nsplit;    // query tiles [0, ts) are split nsplit ways over their positions, the others are not
  float kq_scale;
  int tile_major;  // CTA order, see the kernel
  int8_t* xq;      // q8_1 output instead of o: int8 [M][nqh][256] ...
  float* xd;       // ... and one scale per 32 values, as f32(f16(d)) (q8_store, src/common.cuh:72-81)
};

// Barrier of the NWG threads' warps that share query rows 32q .. 32q+31.
__device__ __forceinline__ void pair_sync(int q) { asm volatile("bar.sync %0, %1;" ::"r"(1 + q), "n"(32 * NWG) : "memory"); }

// Quantises blocks [B0, B0 + NB) of one query row (256 floats at src, or zeros when src is null)
// to int8 with an f32 scale per 32 dims (src/attn.cu:587-606: v = q * kq_scale, d = amax / 127,
// id = 127 / amax, q8 = rint(v * id)) and stores them in row r of the Q tile (K-major,
// 128B-swizzled); dq[i] = scale of block B0 + i.
template <int B0, int NB>
__device__ __forceinline__ void quantise_q_row(const float* src, float kq_scale, uint8_t* sQ, int r, float (&dq)[NB]) {
#pragma unroll
  for (int bi = 0; bi < NB; bi++) {
    const int b = B0 + bi;
    uint32_t w[8];
    float d = 0.f;
    if (src) {
      float v[32];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 f = *(const float4*)(src + b * 32 + j);
        v[j] = __fmul_rn(f.x, kq_scale);
        v[j + 1] = __fmul_rn(f.y, kq_scale);
        v[j + 2] = __fmul_rn(f.z, kq_scale);
        v[j + 3] = __fmul_rn(f.w, kq_scale);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[j]), fabsf(v[j + 1])), fmaxf(fabsf(v[j + 2]), fabsf(v[j + 3]))));
      }
      d = __fdiv_rn(amax, 127.f);
      const float id = amax > 0.f ? __fdiv_rn(127.f, amax) : 0.f;
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int q0 = __float2int_rn(__fmul_rn(v[4 * j], id)), q1 = __float2int_rn(__fmul_rn(v[4 * j + 1], id));
        const int q2 = __float2int_rn(__fmul_rn(v[4 * j + 2], id)), q3 = __float2int_rn(__fmul_rn(v[4 * j + 3], id));
        w[j] = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) |
               ((uint32_t)(q3 & 0xFF) << 24);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) w[j] = 0;
    }
    dq[bi] = d;
    uint8_t* half = sQ + (b >> 2) * (QT * 128);
    const uint32_t c = 2 * (b & 3);
    *(uint4*)(half + swz128(r, c)) = make_uint4(w[0], w[1], w[2], w[3]);
    *(uint4*)(half + swz128(r, c + 1)) = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// Multiplies OCOLS accumulator columns of this warp's 32 TMEM lanes by f. Rare (the reference max
// of a row moves a few times per call), and deliberately not inlined: inlined, its 32 registers of
// payload sit on top of the live state of the hot loop and push that loop into spills.
__device__ __noinline__ void rescale_o(uint32_t taddr, float f) {
#pragma unroll 1
  for (int c = 0; c < OCOLS / 32; c++) {
    uint32_t v[32];
    tmem_ld32(taddr + c * 32, v);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
    tmem_st32(taddr + c * 32, v);
  }
}

// Descriptors of the 32-byte k-block b of a K-major 128B-swizzled int8 tile made of two halves
// of `rows` rows x 128 B.
__device__ __forceinline__ uint64_t desc_kblock(uint32_t tile_addr, int rows, int b) {
  return umma_desc_sw128(tile_addr + (b >> 2) * (rows * 128) + (b & 3) * 32, 16, 1024);
}

__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_i8_kernel(const __grid_constant__ CUtensorMap tm_kv, const __grid_constant__ CUtensorMap tm_ks,
                  const __grid_constant__ CUtensorMap tm_vv, const __grid_constant__ CUtensorMap tm_vs,
                  const PrefillParams p) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  uint64_t* bar = (uint64_t*)(sgen + OFF_BAR);
  uint32_t* tmem_slot = (uint32_t*)(sgen + OFF_MISC);
  volatile int* abort_flag = (volatile int*)(sgen + OFF_MISC + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // CTA order: the query tiles with the most positions first (src/attn.cu:567). tile_major: and that
  // across all heads (block L = head L % nqh of tile rank L / nqh), which matters on a short prefix,
  // where the tiles differ a lot in length and the longest tiles of the last heads would start last.
  // Otherwise head by head (block L = tile rank L % n_tiles of head L / n_tiles), so that the CTAs
  // that run at the same time stream the same K/V rows and share them in L2 (measured: 7 % at 32k).
  // The unsplit CTAs (tiles >= ts) come first, then the pieces of the split tiles, split index slowest.
  int L = (int)blockIdx.x, z = 0, nsplit = 1, ntl = (p.M + QT - 1) / QT - p.ts, tile_base = p.ts;
  if (L >= ntl * p.nqh) {
    L -= ntl * p.nqh;
    ntl = p.ts;
    tile_base = 0;
    nsplit = p.nsplit;
    z = L / (ntl * p.nqh);
    L -= z * ntl * p.nqh;
  }
  const int h = p.tile_major ? L % p.nqh : L / ntl, kh = h / GQA;
  const int t0 = (tile_base + ntl - 1 - (p.tile_major ? L / p.nqh : L % ntl)) * QT;
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
    for (int s = 0; s < 2; s++) {
      mbar_init(&bar[B_KFULL + s], 1);
      mbar_init(&bar[B_KEMPTY + s], N_CONV_WARPS + 1);
      mbar_init(&bar[B_VFULL + s], 1);
      mbar_init(&bar[B_VEMPTY + s], N_CONV_WARPS);
      mbar_init(&bar[B_VFFULL + s], N_CONV_WARPS);
      mbar_init(&bar[B_VFEMPTY + s], 1);
      mbar_init(&bar[B_DKEMPTY + s], N_SOFTMAX_WARPS);
      mbar_init(&bar[B_PFULL + s], N_SOFTMAX_WARPS);
      mbar_init(&bar[B_PEMPTY + s], 1);
    }
    for (int s = 0; s < 4; s++) {
      mbar_init(&bar[B_SFULL + s], 1);
      mbar_init(&bar[B_SEMPTY + s], N_SOFTMAX_WARPS);
    }
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
    const float* dqs = (const float*)(sgen + OFF_DQ) + r;  // block b of this row at dqs[b * QT]
    {
      // this thread quantises 8 / NWG blocks of its row; the scales go through shared memory
      constexpr int NB = 8 / NWG;
      float dqh[NB];
      const float* src = live ? p.qn + ((size_t)t * p.nqh + h) * AD : nullptr;
      if (NWG == 2) {
        if (wg == 0) quantise_q_row<0, NB>(src, p.kq_scale, sgen + OFF_Q, r, dqh);
        else quantise_q_row<NB, NB>(src, p.kq_scale, sgen + OFF_Q, r, dqh);
      } else {
        if (wg == 0) quantise_q_row<0, NB>(src, p.kq_scale, sgen + OFF_Q, r, dqh);
        else if (wg == 1) quantise_q_row<NB, NB>(src, p.kq_scale, sgen + OFF_Q, r, dqh);
        else if (wg == 2) quantise_q_row<(2 * NB) % 8, NB>(src, p.kq_scale, sgen + OFF_Q, r, dqh);
        else quantise_q_row<(3 * NB) % 8, NB>(src, p.kq_scale, sgen + OFF_Q, r, dqh);
      }
#pragma unroll
      for (int i = 0; i < NB; i++) *(float*)(sgen + OFF_DQ + ((NB * wg + i) * QT + r) * 4) = dqh[i];
      fence_proxy_async();
      pair_sync(q);
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_QFULL]);
    }

    const uint32_t tlane = tmem + ((uint32_t)(q * 32) << 16);
    const int limit = pos0 + t + 1;    // positions < limit are visible
    const int col0 = wg * WCOLS;       // this thread's positions of a tile: col0 .. col0 + WCOLS - 1
    float m_run = M_INIT, m_ref = M_INIT;
    uint64_t l2 = pack2(0.f, 0.f);
    const uint64_t log2e2 = pack2(LOG2E, LOG2E);

#pragma unroll 1
    for (int j = 0; j < nt; j++) {
      const int pb = j & 1, ph = (j >> 1) & 1;
      const int p_tile = (it0 + j) * PT;
      mbar_wait(&bar[B_VFFULL + pb], ph, abort_flag, p.status);  // K scale table of this tile is ready
      const uint8_t* dkf = sgen + OFF_DKF + pb * DKF_BYTES;
      uint64_t s2[WCOLS / 2];
#pragma unroll
      for (int i = 0; i < WCOLS / 2; i++) s2[i] = pack2(0.f, 0.f);
#pragma unroll
      for (int b = 0; b < 8; b++) {
        const int slot = b & 3;
#ifdef Q27B_PF_COMMIT_EACH
        mbar_wait(&bar[B_SFULL + slot], (b >> 2) & 1, abort_flag, p.status);
#else
        // (blocks are committed in pairs: the barrier of the pair's second slot covers both)
        mbar_wait(&bar[B_SFULL + (slot | 1)], (b >> 2) & 1, abort_flag, p.status);
#endif
        tc_fence_after();
        // The accumulators come in two halves of 16 columns: 16 registers fewer are live at a time
        // than with one 32-column load, and this kernel runs at its register limit.
        const float dqv = dqs[b * QT];  // this row's Q scale of block b (shared memory: eight registers fewer)
        const uint64_t dqb = pack2(dqv, dqv);
#pragma unroll
        for (int hf = 0; hf < WCOLS / 16; hf++) {
          uint32_t v[16];
          tmem_ld16(tlane + TM_S + slot * PT + col0 + 16 * hf, v);
          tc_wait_ld();
          if (hf == WCOLS / 16 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar[B_SEMPTY + slot]);  // the slot is in registers: it can be overwritten
          }
          const ulonglong2* dk2 = (const ulonglong2*)(dkf + (b * PT + col0 + 16 * hf) * 4);
#pragma unroll
          for (int i = 0; i < 4; i++) {
            const ulonglong2 dk = dk2[i];  // K scales of positions 4i .. 4i+3 (block b)
            // int32 -> f32 is exact here (|sum| <= 32 * 127 * 127 < 2^24)
            const uint64_t f0 = pack2(__int2float_rn((int)v[4 * i]), __int2float_rn((int)v[4 * i + 1]));
            const uint64_t f1 = pack2(__int2float_rn((int)v[4 * i + 2]), __int2float_rn((int)v[4 * i + 3]));
            s2[8 * hf + 2 * i] = fma2(mul2(dqb, dk.x), f0, s2[8 * hf + 2 * i]);
            s2[8 * hf + 2 * i + 1] = fma2(mul2(dqb, dk.y), f1, s2[8 * hf + 2 * i + 1]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_DKEMPTY + pb]);

      // causal mask (only tiles that reach past the first row's limit need it) and this thread's max
      float s[WCOLS];
#pragma unroll
      for (int i = 0; i < WCOLS / 2; i++) unpack2(s2[i], s[2 * i], s[2 * i + 1]);
      float mt = -INFINITY;
      if (p_tile + PT > pos0 + t0 + 1) {
#pragma unroll
        for (int i = 0; i < WCOLS; i++) {
          if (p_tile + col0 + i >= limit) s[i] = -INFINITY;
          mt = fmaxf(mt, s[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < WCOLS; i++) mt = fmaxf(mt, s[i]);
      }
      // row maximum over the NWG threads of the row; the buffer alternates with the tile so that a
      // fast thread cannot overwrite what a partner has not read yet
      xch[(pb * NWG + wg) * QT + r] = mt;
      pair_sync(q);
#pragma unroll
      for (int o = 1; o < NWG; o++) mt = fmaxf(mt, xch[(pb * NWG + ((wg + o) % NWG)) * QT + r]);
      m_run = fmaxf(m_run, mt);

      // Move the reference max when the true max has run away from it (and on the first tile). All
      // threads of a row hold the same m_run and m_ref, so all their warps take the same branch.
      const bool want = m_run > m_ref + TAU;
      if (__any_sync(0xffffffffu, want)) {
        const float f = ex2((m_ref - m_run) * LOG2E);  // 0 on the first move (m_ref = -1e30)
        m_ref = m_run;
        l2 = mul2(l2, pack2(f, f));
        if (j > 0) {
          // O holds the sum of tiles < j once the P V of tile j-1 has completed. This warp rescales
          // columns OCOLS wg .. OCOLS wg + OCOLS - 1 of its 32 rows.
          mbar_wait(&bar[B_PEMPTY + ((j - 1) & 1)], ((j - 1) >> 1) & 1, abort_flag, p.status);
          tc_fence_after();
          rescale_o(tlane + TM_O + wg * OCOLS, f);
          tc_wait_st();
          tc_fence_before();
        }
      }

      // P = exp(s - m_ref): f32 row sum, f16 part of the tile for the P V MMA (WCOLS / 8 chunks of the row)
      mbar_wait(&bar[B_PEMPTY + pb], ph ^ 1, abort_flag, p.status);
      uint8_t* sP = sgen + OFF_P + pb * P_BYTES;
      const float nmb = -m_ref * LOG2E;
      const uint64_t nmb2 = pack2(nmb, nmb);
#pragma unroll
      for (int c = 0; c < WCOLS / 8; c++) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          float a0, a1;
          unpack2(fma2(pack2(s[c * 8 + 2 * k], s[c * 8 + 2 * k + 1]), log2e2, nmb2), a0, a1);
          const float e0 = ex2(a0), e1 = ex2(a1);
          l2 = add2(l2, pack2(e0, e1));
          w[k] = pack_h2(e0, e1);
        }
        *(uint4*)(sP + swz128(r, (WCOLS / 8) * wg + c)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_PFULL + pb]);
    }

    // ---- epilogue: O / l * sigmoid(gate), or the unnormalised partial of this split; this thread
    // writes columns OCOLS wg .. OCOLS wg + OCOLS - 1 of its row
    float la, lb;
    unpack2(l2, la, lb);
    float l = la + lb;
    xch[((nt & 1) * NWG + wg) * QT + r] = l;
    pair_sync(q);
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
    for (int c = 0; c < OCOLS / 32; c++) {
      const int d0 = wg * OCOLS + c * 32;
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
        float* dst = p.xq ? nullptr : p.o + ((size_t)t * p.nqh + h) * AD + d0;
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 gg = *(const float4*)(gt + i);
          float4 y;
          y.x = (__uint_as_float(v[i]) * inv_l) * (1.0f / (1.0f + __expf(-gg.x)));
          y.y = (__uint_as_float(v[i + 1]) * inv_l) * (1.0f / (1.0f + __expf(-gg.y)));
          y.z = (__uint_as_float(v[i + 2]) * inv_l) * (1.0f / (1.0f + __expf(-gg.z)));
          y.w = (__uint_as_float(v[i + 3]) * inv_l) * (1.0f / (1.0f + __expf(-gg.w)));
          if (dst) {
            *(float4*)(dst + i) = y;
          } else {  // keep the values for the q8_1 block below (these 32 columns are exactly one block)
            v[i] = __float_as_uint(y.x); v[i + 1] = __float_as_uint(y.y);
            v[i + 2] = __float_as_uint(y.z); v[i + 3] = __float_as_uint(y.w);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(y.x), fabsf(y.y)), fmaxf(fabsf(y.z), fabsf(y.w))));
          }
        }
        if (!dst) {
          // q8_1 as the reference's quantize_q8_1 / q8_store (src/common.cuh:72-81): d = amax / 127,
          // q = round(y / d) (half away from zero), the scale leaves as f32(f16(d)); IEEE division
          const float dd = __fdiv_rn(amax, 127.0f);
          const size_t oi = ((size_t)t * p.nqh + h) * AD + d0;
          uint32_t w[8];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            uint32_t b[4];
#pragma unroll
            for (int k = 0; k < 4; k++)
              b[k] = amax == 0.0f ? 0u : (uint32_t)(uint8_t)(int8_t)roundf(__fdiv_rn(__uint_as_float(v[i + k]), dd));
            w[i / 4] = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
          }
          *(uint4*)(p.xq + oi) = make_uint4(w[0], w[1], w[2], w[3]);
          *(uint4*)(p.xq + oi + 16) = make_uint4(w[4], w[5], w[6], w[7]);
          p.xd[oi / 32] = __half2float(__float2half_rn(dd));
        }
      }
    }
    tc_fence_before();
  } else if (warp < TMA_WARP) {
    // ================================================================ converter warps
    const int ct = tid - CONV_WARP0 * 32;
    static_assert(N_CONV_THREADS == 128, "the item mapping below is for 128 converter threads");
    const int cv_row0 = (2 * (ct >> 5)) ^ (5 * ((ct >> 2) & 1)), cv_c16 = (ct & 3) + 4 * ((ct >> 3) & 3);
    const uint32_t cv_src = (cv_c16 >> 3) * (PT * 128) + swz128(cv_row0, cv_c16 & 7);
    const uint32_t cv_sc = 2 * PT * 128 + cv_row0 * 16 + (cv_c16 >> 1) * 2;
    const uint32_t cv_dst = (cv_c16 >> 2) * (PT * 128) + swz128(cv_row0, 2 * (cv_c16 & 3));
    for (int j = 0; j < nt; j++) {
      const int pb = j & 1, ph = (j >> 1) & 1;
      mbar_wait(&bar[B_VFULL + pb], ph, abort_flag, p.status);
      mbar_wait(&bar[B_KFULL + pb], ph, abort_flag, p.status);
      mbar_wait(&bar[B_VFEMPTY + pb], ph ^ 1, abort_flag, p.status);
      mbar_wait(&bar[B_DKEMPTY + pb], ph ^ 1, abort_flag, p.status);
      const uint8_t* vst = sgen + OFF_V + pb * KST_PAD;
      const uint8_t* kst = sgen + OFF_K + pb * KST_PAD;
      uint8_t* vf = sgen + OFF_VF + pb * VF_BYTES;
      // V: 64 rows x 16 chunks of 16 int8 -> 16 f16 (one rounding of q * d, as src/attn.cu:59-76).
      // Item = (row, 16-dim chunk); eight neighbouring lanes take 4 chunks of rows rho and rho ^ 5,
      // which keeps both the swizzled 16-byte loads and the swizzled 16-byte stores conflict-free.
      // A thread owns the same chunk of rows row0, row0 + 8, ..: rows 8 apart share their swizzle
      // phase, so every address is a per-thread base (computed before the tile loop) plus a constant.
#pragma unroll 1
      for (int k0 = 0; k0 < 1024 / N_CONV_THREADS; k0 += 4) {
        // Loads of four items first: a shared-memory load cannot be moved above an earlier store, so
        // load / convert / store per item would serialise the load latencies.
        uint4 x[4];
        __half d[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          x[k] = *(const uint4*)(vst + cv_src + (k0 + k) * 1024);
          d[k] = *(const __half*)(vst + cv_sc + (k0 + k) * 128);
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
          if ((it0 + j) * PT + cv_row0 + 8 * (k0 + k) >= n_end) {  // rows past the end may hold anything: P is 0 there, V must be too
#pragma unroll
            for (int w = 0; w < 8; w++) o[w] = 0;
          }
          uint8_t* dst = vf + (k0 + k) * 1024;
          *(uint4*)(dst + cv_dst) = make_uint4(o[0], o[1], o[2], o[3]);
          *(uint4*)(dst + (cv_dst ^ 16u)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
      // K scales f16 [64][8] -> f32 [8][64]
      {
        float* dkf = (float*)(sgen + OFF_DKF + pb * DKF_BYTES);
#pragma unroll
        for (int u = ct; u < 128; u += N_CONV_THREADS) {
          const int row = u >> 1, b0 = (u & 1) * 4;
          const uint2 sc = *(const uint2*)(kst + 2 * PT * 128 + row * 16 + b0 * 2);
          const __half2 s01 = u32_as_h2(sc.x), s23 = u32_as_h2(sc.y);
          dkf[(b0 + 0) * PT + row] = __low2float(s01);
          dkf[(b0 + 1) * PT + row] = __high2float(s01);
          dkf[(b0 + 2) * PT + row] = __low2float(s23);
          dkf[(b0 + 3) * PT + row] = __high2float(s23);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bar[B_VFFULL + pb]);
        mbar_arrive(&bar[B_VEMPTY + pb]);
        mbar_arrive(&bar[B_KEMPTY + pb]);
      }
    }
  } else if (warp == TMA_WARP) {
    // ================================================================ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_kv);
      tma_prefetch_desc(&tm_ks);
      tma_prefetch_desc(&tm_vv);
      tma_prefetch_desc(&tm_vs);
      for (int j = 0; j < nt; j++) {
        const int pb = j & 1, ph = (j >> 1) & 1;
        const int row = kh * p.n_ctx + (it0 + j) * PT;
        uint8_t* kst = sgen + OFF_K + pb * KST_PAD;
        uint8_t* vst = sgen + OFF_V + pb * KST_PAD;
        mbar_wait(&bar[B_KEMPTY + pb], ph ^ 1, abort_flag, p.status);
        mbar_expect_tx(&bar[B_KFULL + pb], KST_BYTES);
        tma_load_2d(kst, &tm_kv, 0, row, &bar[B_KFULL + pb]);
        tma_load_2d(kst + PT * 128, &tm_kv, 128, row, &bar[B_KFULL + pb]);
        tma_load_2d(kst + 2 * PT * 128, &tm_ks, 0, row, &bar[B_KFULL + pb]);
        mbar_wait(&bar[B_VEMPTY + pb], ph ^ 1, abort_flag, p.status);
        mbar_expect_tx(&bar[B_VFULL + pb], KST_BYTES);
        tma_load_2d(vst, &tm_vv, 0, row, &bar[B_VFULL + pb]);
        tma_load_2d(vst + PT * 128, &tm_vv, 128, row, &bar[B_VFULL + pb]);
        tma_load_2d(vst + 2 * PT * 128, &tm_vs, 0, row, &bar[B_VFULL + pb]);
      }
    }
  } else {
    // ================================================================ MMA issuer
    if (lane == 0) {
      mbar_wait(&bar[B_QFULL], 0, abort_flag, p.status);
      tc_fence_after();
      auto issue_pv = [&](int jj) {
        const int pb = jj & 1, ph = (jj >> 1) & 1;
        mbar_wait(&bar[B_PFULL + pb], ph, abort_flag, p.status);
        mbar_wait(&bar[B_VFFULL + pb], ph, abort_flag, p.status);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < PT / 16; kk++) {
          const uint64_t da = umma_desc_sw128(sbase + OFF_P + pb * P_BYTES + kk * 32, 16, 1024);
          const uint64_t db = umma_desc_sw128(sbase + OFF_VF + pb * VF_BYTES + kk * 2048, PT * 128, 1024);
          tc_mma_f16(tmem + TM_O, da, db, IDESC_PV, (jj > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(&bar[B_PEMPTY + pb]);
        tc_commit(&bar[B_VFEMPTY + pb]);
      };
      for (int j = 0; j < nt; j++) {
        const int pb = j & 1, ph = (j >> 1) & 1;
        mbar_wait(&bar[B_KFULL + pb], ph, abort_flag, p.status);
        tc_fence_after();
#pragma unroll
        for (int b = 0; b < 8; b++) {
          const int slot = b & 3;
          mbar_wait(&bar[B_SEMPTY + slot], ((b >> 2) & 1) ^ 1, abort_flag, p.status);
          tc_fence_after();
          tc_mma_i8(tmem + TM_S + slot * PT, desc_kblock(sbase + OFF_Q, QT, b),
                    desc_kblock(sbase + OFF_K + pb * KST_PAD, PT, b), IDESC_QK, 0u);
#ifdef Q27B_PF_COMMIT_EACH
          tc_commit(&bar[B_SFULL + slot]);
#else
          // One commit per two blocks: an MMA followed by its own commit costs the issuing thread the better
          // part of a thousand cycles (measured on the decode kernel with P V on tcgen05), eight of them per
          // tile were most of a tile's time here.
          if (b & 1) tc_commit(&bar[B_SFULL + slot]);
#endif
        }
        tc_commit(&bar[B_KEMPTY + pb]);
        if (j >= 1) issue_pv(j - 1);
      }
      issue_pv(nt - 1);
      tc_commit(&bar[B_ODONE]);
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

// ---------------------------------------------------------------- integer-stage test hook
// 128 threads: quantise up to 128 rows, load one 64-row K tile by TMA, run the 8 block MMAs into
// 8 x 64 TMEM columns, dump everything.
struct QkDebugParams {
  const float* x;
  int rows;
  float kq_scale;
  int row0;   // first row of the K tile in the cache's row space
  int npos;
  int8_t* q_i8;
  float* q_scale;
  int32_t* acc;
  int* status;
};
constexpr int DBG_OFF_K = SQ_BYTES;
constexpr int DBG_OFF_BAR = DBG_OFF_K + 2 * PT * 128;
constexpr int DBG_SMEM = DBG_OFF_BAR + 64 + 1024;

__global__ void __launch_bounds__(128, 1)
prefill_qk_debug_kernel(const __grid_constant__ CUtensorMap tm_kv, const QkDebugParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  uint64_t* bar = (uint64_t*)(sgen + DBG_OFF_BAR);
  uint32_t* tmem_slot = (uint32_t*)(sgen + DBG_OFF_BAR + 32);
  volatile int* abort_flag = (volatile int*)(sgen + DBG_OFF_BAR + 36);
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    *abort_flag = 0;
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

  float dq[8];
  quantise_q_row<0, 8>(tid < p.rows ? p.x + (size_t)tid * AD : nullptr, p.kq_scale, sgen, tid, dq);
  if (tid < p.rows) {
    for (int b = 0; b < 8; b++) p.q_scale[tid * 8 + b] = dq[b];
    for (int b = 0; b < 8; b++)
      for (int c = 0; c < 2; c++) {
        const uint4 w = *(const uint4*)(sgen + (b >> 2) * (QT * 128) + swz128(tid, 2 * (b & 3) + c));
        *(uint4*)(p.q_i8 + (size_t)tid * AD + b * 32 + c * 16) = w;
      }
  }
  fence_proxy_async();
  __syncthreads();
  if (tid == 0) {
    mbar_expect_tx(&bar[0], 2 * PT * 128);
    tma_load_2d(sgen + DBG_OFF_K, &tm_kv, 0, p.row0, &bar[0]);
    tma_load_2d(sgen + DBG_OFF_K + PT * 128, &tm_kv, 128, p.row0, &bar[0]);
    mbar_wait(&bar[0], 0, abort_flag, p.status);
    tc_fence_after();
    for (int b = 0; b < 8; b++)
      tc_mma_i8(tmem + b * PT, desc_kblock(sbase, QT, b), desc_kblock(sbase + DBG_OFF_K, PT, b), IDESC_QK, 0u);
    tc_commit(&bar[1]);
  }
  mbar_wait(&bar[1], 0, abort_flag, p.status);
  tc_fence_after();
  const uint32_t tlane = tmem + ((uint32_t)(warp * 32) << 16);
  for (int b = 0; b < 8; b++)
    for (int hf = 0; hf < 2; hf++) {
      uint32_t v[32];
      tmem_ld32(tlane + b * PT + hf * 32, v);
      tc_wait_ld();
      if (tid < p.rows)
        for (int i = 0; i < 32; i++) {
          const int pp = hf * 32 + i;
          if (pp < p.npos) p.acc[((size_t)tid * p.npos + pp) * 8 + b] = (int32_t)v[i];
        }
    }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

int prefill_setup(DeviceCtx* ctx) {
  if (!ctx->prefill_attr) {
    Q27B_CK(cudaFuncSetAttribute(prefill_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM_BYTES));
    Q27B_CK(cudaFuncSetAttribute(prefill_qk_debug_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DBG_SMEM));
    ctx->prefill_attr = true;
  }
  return Q27B_OK;
}

}  // namespace

}  // namespace q27b

using namespace q27b;

// Which kernel serves a q8_0 cache: int8 Q K^T (default, as the reference since its Q27_ATTN_I8
// default) or the f16-QK kernel on dequantised K and V (the reference's Q27_ATTN_I8=0).
static std::atomic<int> g_prefill_choice{-1};  // -1: not read yet; 0 default, 1 int8 Q K^T, 2 f16 Q K^T
static bool use_f16_qk() {
  int k = g_prefill_choice.load(std::memory_order_relaxed);
  if (k < 0) {
    const char* e = getenv("Q27_ATTN_I8");
    k = e && e[0] == '0' ? 2 : 0;
    int expected = -1;
    if (!g_prefill_choice.compare_exchange_strong(expected, k)) k = expected;
  }
  return k == 2;
}

extern "C" {

int q27b_prefill_split_plan(int M, int nqh, int n_sm, int depth_hint, int* split_tiles, int* pieces) {
  if (M < 1 || nqh < 1 || n_sm < 1 || !split_tiles || !pieces) return fail(Q27B_BAD_SHAPE, "prefill_split_plan: bad argument");
  const SplitPlan sp = plan_prefill_split((M + QT - 1) / QT, nqh, n_sm, M, depth_hint, false);
  *split_tiles = sp.ts;
  *pieces = sp.ns;
  return Q27B_OK;
}

int q27b_set_prefill_kernel(int which) {
  if (which < 0 || which > 2) return fail(Q27B_BAD_SHAPE, "set_prefill_kernel: 0 auto, 1 int8 QK, 2 f16 QK");
  g_prefill_choice.store(which);
  return Q27B_OK;
}

static int prefill_impl(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o, int8_t* xq,
                        float* xd, const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx, int q8,
                        void* stream, int depth_hint) {
  if (nkvh < 1 || nqh != nkvh * GQA || M < 1 || n_ctx < 1) return fail(Q27B_BAD_SHAPE, "attn_prefill: bad shape");
  if (!qn || !qg || !kcache || !vcache || (!o && !xq) || (xq && !xd) || !pos0)
    return fail(Q27B_BAD_SHAPE, "attn_prefill: null pointer");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  if (!q8 || use_f16_qk())  // the f16-QK kernel (the reference's attn_prefill_kernel<PT, Q8>, src/attn.cu:338-528)
    return launch_prefill_f16(ctx, qn, qg, kcache, vcache, o, xq, xd, pos0, M, kq_scale, nqh, nkvh, n_ctx, q8 != 0,
                              depth_hint, (cudaStream_t)stream);
  if (int rc = prefill_setup(ctx)) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  const int tiles = (M + QT - 1) / QT;
  SplitPlan sp = plan_prefill_split(tiles, nqh, ctx->n_sm, M, depth_hint, false);
  float* part;  // the fixed prefill workspace; the plan is cut to what it holds
  if (int rc = fit_prefill_split(ctx, &sp.ts, &sp.ns, M, nqh, false, &part)) return rc;
  const int nsplit = sp.ns, Ms = std::min(M, sp.ts * QT);
  CUtensorMap kvm, ksm, vvm, vsm;
  if (int rc = q8_tmaps(kcache, (uint64_t)nkvh * n_ctx, &kvm, &ksm)) return rc;
  if (int rc = q8_tmaps(vcache, (uint64_t)nkvh * n_ctx, &vvm, &vsm)) return rc;
  const CUtensorMap *kv = &kvm, *ks = &ksm, *vv = &vvm, *vs = &vsm;
  PrefillParams p = {};
  p.qn = qn; p.qg = qg; p.o = o; p.xq = xq; p.xd = xd; p.part = nsplit > 1 ? part : nullptr; p.pos0 = pos0; p.status = ctx->status;
  p.M = M; p.nqh = nqh; p.nkvh = nkvh; p.n_ctx = n_ctx; p.ts = sp.ts; p.nsplit = nsplit; p.kq_scale = kq_scale;
  p.tile_major = depth_hint >= 0 && depth_hint < 4 * M;  // short prefix: the causal part dominates
  prefill_i8_kernel<<<(tiles - sp.ts) * nqh + sp.ts * nqh * nsplit, PF_THREADS, PF_SMEM_BYTES, s>>>(*kv, *ks, *vv, *vs, p);
  Q27B_CK(cudaGetLastError());
  if (nsplit > 1) {  // the split tokens are rows [0, Ms * nqh) of every array
    MergeParams mp = {};
    mp.part = part; mp.nparts = nsplit; mp.part_stride = (int64_t)Ms * nqh * PROW; mp.rows = (int64_t)Ms * nqh;
    mp.qg = qg; mp.o = o; mp.xq = xq; mp.xd = xd;
    return launch_merge(mp, false, s);
  }
  return Q27B_OK;
}

int q27b_attn_prefill(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                      const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, void* stream,
                      int depth_hint) {
  if (!o) return fail(Q27B_BAD_SHAPE, "attn_prefill: null pointer");
  return prefill_impl(qn, qg, kcache, vcache, o, nullptr, nullptr, pos0, M, kq_scale, nqh, nkvh, n_ctx, q8, stream, depth_hint);
}

int q27b_attn_prefill_q8_1(const float* qn, const float* qg, const void* kcache, const void* vcache, int8_t* xq, float* xd,
                           const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, void* stream,
                           int depth_hint) {
  if (!xq || !xd) return fail(Q27B_BAD_SHAPE, "attn_prefill: null pointer");
  return prefill_impl(qn, qg, kcache, vcache, nullptr, xq, xd, pos0, M, kq_scale, nqh, nkvh, n_ctx, q8, stream, depth_hint);
}

int q27b_prefill_qk_debug(const float* x, int rows, float kq_scale, const void* kcache, int nkvh, int n_ctx, int kh,
                          int p0, int npos, int8_t* q_i8, float* q_scale, int32_t* acc, void* stream) {
  if (rows < 1 || rows > QT || npos < 1 || npos > PT || kh < 0 || kh >= nkvh || p0 < 0 || p0 + npos > n_ctx)
    return fail(Q27B_BAD_SHAPE, "prefill_qk_debug: bad shape");
  if (!x || !kcache || !q_i8 || !q_scale || !acc) return fail(Q27B_BAD_SHAPE, "prefill_qk_debug: null pointer");
  DeviceCtx* ctx;
  if (int rc = device_ctx(&ctx)) return rc;
  if (int rc = prefill_setup(ctx)) return rc;
  CUtensorMap kvm, ksm;
  if (int rc = q8_tmaps(kcache, (uint64_t)nkvh * n_ctx, &kvm, &ksm)) return rc;
  const CUtensorMap* kv = &kvm;
  QkDebugParams p = {x, rows, kq_scale, kh * n_ctx + p0, npos, q_i8, q_scale, acc, ctx->status};
  prefill_qk_debug_kernel<<<1, 128, DBG_SMEM, (cudaStream_t)stream>>>(*kv, p);
  Q27B_CK(cudaGetLastError());
  return Q27B_OK;
}

}  // extern "C"
