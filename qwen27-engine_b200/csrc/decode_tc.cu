// Split-K flash-decode over a q8_0 KV cache with both contractions on the 5th-generation tensor
// cores (tcgen05.mma kind::f16, accumulators in TMEM).
//
// Same operator, same work decomposition, same partial layout and same roundings as the warp-MMA
// kernel in decode.cu (reference: attn_mma_kernel, src/attn.cu:95-292): Q * scale -> f16,
// K / V -> f16(int8 * f16 scale), P -> f16, f32 accumulation, row sums from the f32 P.
// Why a second kernel: measured on B200, the legacy mma.sync path shares its issue bandwidth with
// the int8 -> f16 conversion arithmetic (one group of four warps alone reaches 86 % of the
// throughput of two), so the warp-MMA kernel is bound by instruction issue at about 5 TB/s. Here
// the SIMT lanes only dequantise; everything else is asynchronous hardware:
//
//   warp 12     one lane: TMA of 64-position raw tiles (int8 values + f16 scales) into a 4-stage ring.
//   warps 0-7   converters: raw tile -> f16 K tile and f16 V tile in shared memory, both as
//               [64-dim segment][position][128 B] with the 128-byte swizzle. Read as "K-major" this
//               is the A operand K[p][d] of S^T = K Q^T; read as "MN-major" it is the A operand
//               V^T[d][p] of O^T = V^T P^T. No transpose, no fragment shuffling.
//   warp 13     one lane: issues the MMAs. S^T (positions on the 128 TMEM lanes, of which 64 are
//               used; the 6T query rows on 32 columns) = 16 x (128x32x16); O^T (head dims on the
//               lanes, two halves of 128; query rows on the columns) += 2 x 4 x (128x32x16).
//   warps 8-11  softmax group. Warps 8 and 9 own one position each per lane: they read their row
//               of S^T from TMEM, form P = exp(S - m) against the reference maxima m[r] (moved only
//               when a score exceeds them by more than TAU), keep per-lane partial row sums, and
//               write P^T (f16, [query row][position], swizzled) for the second MMA. All four warps
//               rescale O^T in TMEM on the rare tiles where m moves, and write the partial at the end.
// TMEM: columns 0-31 and 32-63 two S^T buffers, 64-95 and 96-127 the two halves of O^T.
#include "common.cuh"
#include "decode_params.h"

namespace q27b {
namespace {

constexpr int TILE = 64;                    // positions per tile
constexpr int NST = 4;                      // raw stages
constexpr int RAW_BYTES = 2 * TILE * AD + 2 * TILE * 16;  // 34816: K values, V values, K scales, V scales
constexpr int R_KV = 0, R_VV = TILE * AD, R_KS = 2 * TILE * AD, R_VS = 2 * TILE * AD + TILE * 16;
constexpr int SEG = TILE * 128;             // one 64-dim segment of an f16 tile: [64 positions][128 B]
constexpr int F16_TILE = 4 * SEG;           // 32 KB
constexpr int QSEG = 32 * 128;              // one 64-dim segment of Q^T: [32 rows][128 B]
constexpr int P_BYTES = 32 * 128;           // P^T: [32 query rows][64 positions] f16
constexpr int OFF_RAW = 0;
constexpr int OFF_KF = OFF_RAW + NST * RAW_BYTES;
constexpr int OFF_VF = OFF_KF + F16_TILE;
constexpr int OFF_Q = OFF_VF + F16_TILE;
constexpr int OFF_PB = OFF_Q + 4 * QSEG;    // two buffers
constexpr int OFF_X = OFF_PB + 2 * P_BYTES; // softmax exchange area (floats): colmax [2][24], f [24], l [2][24], m [24], tokens [2]
constexpr int X_CMAX = 0, X_F = 48, X_L = 72, X_M = 120, X_TOK = 144;
constexpr int OFF_BAR = OFF_X + 160 * 4;
constexpr int NBAR = 2 * NST + 4 + 8 + 2;   // raw full/empty, kf/vf full/empty, s/p full/empty x2, q_full, o_done
constexpr int OFF_MISC = OFF_BAR + NBAR * 8;
constexpr int TC_SMEM_USED = OFF_MISC + 16;
constexpr int TC_SMEM_BYTES = TC_SMEM_USED + 1024;
static_assert(OFF_KF % 1024 == 0 && OFF_VF % 1024 == 0 && OFF_Q % 1024 == 0 && OFF_PB % 1024 == 0, "swizzled tiles need 1024-byte alignment");
static_assert(TC_SMEM_BYTES <= 232448, "shared memory budget of one CTA");

enum {
  B_RAWFULL = 0,             // [NST]
  B_RAWEMPTY = NST,          // [NST]
  B_KFFULL = 2 * NST,
  B_KFEMPTY = 2 * NST + 1,
  B_VFFULL = 2 * NST + 2,
  B_VFEMPTY = 2 * NST + 3,
  B_SFULL = 2 * NST + 4,     // [2]
  B_SEMPTY = 2 * NST + 6,    // [2]
  B_PFULL = 2 * NST + 8,     // [2]
  B_PEMPTY = 2 * NST + 10,   // [2]
  B_QFULL = 2 * NST + 12,
  B_ODONE = 2 * NST + 13,
};

constexpr int N_CONV_WARPS = 8, SM_WARP0 = 8, TMA_WARP = 12, MMA_WARP = 13;
constexpr int TC_THREADS = 14 * 32;
constexpr int BAR_SM = 1;                   // named barrier of the softmax group (128 threads)
constexpr uint32_t TMEM_COLS = 128;
constexpr uint32_t TM_S = 0, TM_O = 64;
constexpr float TAU = 8.0f;
constexpr uint32_t IDESC_QK = umma_idesc(1, 0, 0, 0, 0, 128, 32);  // f32 += f16 * f16, A and B K-major, M128 N32
constexpr uint32_t IDESC_PV = umma_idesc(1, 0, 0, 1, 0, 128, 32);  // A (V^T) MN-major, B (P^T) K-major

__device__ __forceinline__ void sm_sync() { asm volatile("bar.sync %0, 128;" ::"r"(BAR_SM) : "memory"); }

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

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ch = blockIdx.x, kh = blockIdx.y;
  const int T = p.T, R = GQA * T;
  const int seq = PAGED ? blockIdx.z : 0;
  const int pos0 = PAGED ? p.seq_len[seq] - T : *p.pos0;
  const float* qn = p.qn + (size_t)seq * T * p.nqh * AD;

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
  if (c0 >= c1) {  // empty chunk: neutral partial (src/attn.cu:117-120); the paged merge never reads it
    if (!PAGED)
      for (int i = tid; i < R * PROW; i += TC_THREADS) out[i] = (i % PROW == 0) ? M_INIT : 0.f;
    return;
  }
  const int nt = (c1 - c0 + TILE - 1) / TILE;

  if (tid == 0) {
    for (int s = 0; s < NST; s++) {
      mbar_init(&bar[B_RAWFULL + s], 1);
      mbar_init(&bar[B_RAWEMPTY + s], N_CONV_WARPS);
    }
    mbar_init(&bar[B_KFFULL], N_CONV_WARPS);
    mbar_init(&bar[B_KFEMPTY], 1);
    mbar_init(&bar[B_VFFULL], N_CONV_WARPS);
    mbar_init(&bar[B_VFEMPTY], 1);
    for (int s = 0; s < 2; s++) {
      mbar_init(&bar[B_SFULL + s], 1);
      mbar_init(&bar[B_SEMPTY + s], 2);
      mbar_init(&bar[B_PFULL + s], 2);
      mbar_init(&bar[B_PEMPTY + s], 1);
    }
    mbar_init(&bar[B_QFULL], 4);
    mbar_init(&bar[B_ODONE], 1);
    *abort_flag = 0;
    ((volatile uint32_t*)(xf + X_TOK))[0] = 0;
    ((volatile uint32_t*)(xf + X_TOK))[1] = 0;
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

  if (warp < N_CONV_WARPS) {
    // ================================================================ converters
    // One item = 16 int8 of one row -> 16 f16 (32 bytes = two 16-byte chunks of a segment row). Eight
    // neighbouring lanes take 4 items of rows rho and rho ^ 5, which keeps the swizzled 16-byte loads
    // and stores free of bank conflicts. 1024 items per operand and tile, 4 per thread.
    int it_row[4], it_c16[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int item = tid + 256 * k;
      it_row[k] = (2 * (item >> 5)) ^ (5 * ((item >> 2) & 1));
      it_c16[k] = (item & 3) + 4 * ((item >> 3) & 3);
    }
    auto convert = [&](const uint8_t* vals, const uint8_t* scales, uint8_t* dst, int rows_valid, bool zero_tail) {
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const int row = it_row[k], c16 = it_c16[k];
        const uint4 x = *(const uint4*)(vals + (c16 >> 3) * SEG + swz128(row, c16 & 7));
        const __half d = *(const __half*)(scales + row * 16 + (c16 >> 1) * 2);
        const __half2 dd = __half2half2(d);
        const uint32_t xw[4] = {x.x ^ 0x80808080u, x.y ^ 0x80808080u, x.z ^ 0x80808080u, x.w ^ 0x80808080u};
        uint32_t o[8];
#pragma unroll
        for (int w = 0; w < 4; w++) {
          o[2 * w] = dq_pair(__byte_perm(xw[w], 0x64646464u, 0x4140), dd);
          o[2 * w + 1] = dq_pair(__byte_perm(xw[w], 0x64646464u, 0x4342), dd);
        }
        if (zero_tail && row >= rows_valid) {  // rows past the end may hold anything: P is 0 there, V must be too
#pragma unroll
          for (int w = 0; w < 8; w++) o[w] = 0;
        }
        uint8_t* seg = dst + (c16 >> 2) * SEG;
        const uint32_t cc = 2 * (c16 & 3);
        *(uint4*)(seg + swz128(row, cc)) = make_uint4(o[0], o[1], o[2], o[3]);
        *(uint4*)(seg + swz128(row, cc + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
      }
    };
    for (int j = 0; j < nt; j++) {
      const int st = j % NST;
      const uint8_t* raw = sgen + OFF_RAW + st * RAW_BYTES;
      const int rows_valid = c1 - (c0 + j * TILE);
      mbar_wait(&bar[B_RAWFULL + st], (j / NST) & 1, abort_flag, p.status);
      mbar_wait(&bar[B_KFEMPTY], (j & 1) ^ 1, abort_flag, p.status);
      convert(raw + R_KV, raw + R_KS, sgen + OFF_KF, rows_valid, false);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar[B_KFFULL]);
      mbar_wait(&bar[B_VFEMPTY], (j & 1) ^ 1, abort_flag, p.status);
      convert(raw + R_VV, raw + R_VS, sgen + OFF_VF, rows_valid, rows_valid < TILE);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bar[B_VFFULL]);
        mbar_arrive(&bar[B_RAWEMPTY + st]);
      }
    }
  } else if (warp < TMA_WARP) {
    // ================================================================ softmax group
    const int sw = warp - SM_WARP0;          // TMEM lane quarter
    const int st_tid = tid - SM_WARP0 * 32;  // 0..127
    const bool active = sw < 2;              // owns positions 32 sw + lane of every tile
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

    float m_ref[MAXR], lacc[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; r++) {
      m_ref[r] = M_INIT;
      lacc[r] = 0.f;
    }
    const int lim_base = pos0 + 1 - p.base_pos;  // local rows < lim_base + t are visible to token t
    volatile uint32_t* tok = (volatile uint32_t*)(xf + X_TOK);

    for (int j = 0; j < nt; j++) {
      const int slot = j & 1;
      const int tile_p0 = c0 + j * TILE;
      float s[MAXR];
      if (active) {
        mbar_wait(&bar[B_SFULL + slot], (j >> 1) & 1, abort_flag, p.status);
        tc_fence_after();
        uint32_t v[32];
        tmem_ld32(tlane + TM_S + slot * 32, v);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[B_SEMPTY + slot]);
        const int pos = tile_p0 + sw * 32 + lane;
        bool exceed = j == 0;
#pragma unroll
        for (int r = 0; r < MAXR; r++) {
          s[r] = __uint_as_float(v[r]);
          if (pos >= min(c1, lim_base + min(r / GQA, T - 1))) s[r] = -INFINITY;
          exceed |= s[r] > m_ref[r] + TAU;
        }
        if (__any_sync(0xffffffffu, exceed) && lane == 0) tok[slot] = (uint32_t)(j + 1);
      }
      sm_sync();
      if (tok[slot] == (uint32_t)(j + 1)) {
        // ---- some score ran away from the reference maxima (always on the first tile): move them
        if (active) {
#pragma unroll
          for (int r = 0; r < MAXR; r++) {
            float v = s[r];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (lane == 0) xf[X_CMAX + sw * MAXR + r] = v;
          }
        }
        sm_sync();
        if (active) {
#pragma unroll
          for (int r = 0; r < MAXR; r++) {
            const float mn = fmaxf(m_ref[r], fmaxf(xf[X_CMAX + r], xf[X_CMAX + MAXR + r]));
            const float f = ex2((m_ref[r] - mn) * LOG2E);
            m_ref[r] = mn;
            lacc[r] *= f;
            if (sw == 0 && lane == 0) xf[X_F + r] = f;
          }
        }
        sm_sync();
        if (j > 0) {
          // O^T holds the tiles < j once the second MMA of tile j-1 has completed; every warp of the
          // group rescales its 32 lanes (head dims), column r by f[r].
          mbar_wait(&bar[B_PEMPTY + ((j - 1) & 1)], ((j - 1) >> 1) & 1, abort_flag, p.status);
          tc_fence_after();
#pragma unroll 1
          for (int h = 0; h < 2; h++) {
            uint32_t v[32];
            tmem_ld32(tlane + TM_O + h * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int r = 0; r < MAXR; r++) v[r] = __float_as_uint(__uint_as_float(v[r]) * xf[X_F + r]);
            tmem_st32(tlane + TM_O + h * 32, v);
          }
          tc_wait_st();
          tc_fence_before();
        }
        sm_sync();  // the rescale is complete before anybody releases the next second MMA
      }
      if (active) {
        // P = exp(S - m): per-lane partial row sums; P^T[r][position] as f16 for the second MMA
        mbar_wait(&bar[B_PEMPTY + slot], ((j >> 1) & 1) ^ 1, abort_flag, p.status);
        uint8_t* pb = sgen + OFF_PB + slot * P_BYTES;
        const int pp = sw * 32 + lane;
#pragma unroll
        for (int r = 0; r < MAXR; r++) {
          const float e = ex2(fmaf(s[r], LOG2E, -m_ref[r] * LOG2E));
          lacc[r] += e;
          *(__half*)(pb + r * 128 + ((((uint32_t)pp >> 3) ^ (r & 7)) << 4) + (pp & 7) * 2) = __float2half_rn(e);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar[B_PFULL + slot]);
      }
    }

    // ---- epilogue: row sums over the 64 position lanes, then the partial (m, l, O[256]) per query row
    if (active) {
#pragma unroll
      for (int r = 0; r < MAXR; r++) {
        float v = lacc[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) {
          xf[X_L + sw * MAXR + r] = v;
          if (sw == 0) xf[X_M + r] = m_ref[r];
        }
      }
    }
    sm_sync();
    mbar_wait(&bar[B_ODONE], 0, abort_flag, p.status);
    tc_fence_after();
    if (st_tid < R) {
      out[(size_t)st_tid * PROW] = xf[X_M + st_tid];
      out[(size_t)st_tid * PROW + 1] = xf[X_L + st_tid] + xf[X_L + MAXR + st_tid];
    }
#pragma unroll 1
    for (int h = 0; h < 2; h++) {
      uint32_t v[32];
      tmem_ld32(tlane + TM_O + h * 32, v);
      tc_wait_ld();
      const int d = h * 128 + st_tid;  // TMEM lane = head dim within the half
#pragma unroll
      for (int r = 0; r < MAXR; r++)
        if (r < R) out[(size_t)r * PROW + 2 + d] = __uint_as_float(v[r]);
    }
    tc_fence_before();
  } else if (warp == TMA_WARP) {
    // ================================================================ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_kv);
      tma_prefetch_desc(&tm_ks);
      tma_prefetch_desc(&tm_vv);
      tma_prefetch_desc(&tm_vs);
      const int row0 = kh * p.n_ctx + c0;
      for (int j = 0; j < nt; j++) {
        const int st = j % NST;
        uint8_t* raw = sgen + OFF_RAW + st * RAW_BYTES;
        int row = row0 + j * TILE;
        if (PAGED) {  // a tile never straddles a page (64 | 256)
          const int pp = c0 + j * TILE;
          int pg = p.page_table[(size_t)seq * p.max_pages + pp / Q27B_PAGE];
          if (pg < 0 || pg >= p.n_pages) {  // never read outside the pool: flag it and read page 0
            atomicOr(p.status, ST_BAD_PAGE);
            pg = 0;
          }
          row = (pg * p.nkvh + kh) * Q27B_PAGE + pp % Q27B_PAGE;
        }
        mbar_wait(&bar[B_RAWEMPTY + st], ((j / NST) & 1) ^ 1, abort_flag, p.status);
        mbar_expect_tx(&bar[B_RAWFULL + st], RAW_BYTES);
        tma_load_2d(raw + R_KV, &tm_kv, 0, row, &bar[B_RAWFULL + st]);
        tma_load_2d(raw + R_KV + SEG, &tm_kv, 128, row, &bar[B_RAWFULL + st]);
        tma_load_2d(raw + R_KS, &tm_ks, 0, row, &bar[B_RAWFULL + st]);
        tma_load_2d(raw + R_VV, &tm_vv, 0, row, &bar[B_RAWFULL + st]);
        tma_load_2d(raw + R_VV + SEG, &tm_vv, 128, row, &bar[B_RAWFULL + st]);
        tma_load_2d(raw + R_VS, &tm_vs, 0, row, &bar[B_RAWFULL + st]);
      }
    }
  } else {
    // ================================================================ MMA issuer
    if (lane == 0) {
      mbar_wait(&bar[B_QFULL], 0, abort_flag, p.status);
      tc_fence_after();
      auto issue_pv = [&](int jj) {
        const int slot = jj & 1;
        mbar_wait(&bar[B_PFULL + slot], (jj >> 1) & 1, abort_flag, p.status);
        mbar_wait(&bar[B_VFFULL], jj & 1, abort_flag, p.status);
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
          for (int kk = 0; kk < TILE / 16; kk++) {
            // A = V^T[head dims 128h..][16 positions]: two 64-dim segments (8192 B apart), MN-major
            const uint64_t da = umma_desc_sw128(sbase + OFF_VF + 2 * h * SEG + kk * 2048, SEG, 1024);
            const uint64_t db = umma_desc_sw128(sbase + OFF_PB + slot * P_BYTES + kk * 32, 16, 1024);
            tc_mma_f16(tmem + TM_O + h * 32, da, db, IDESC_PV, (jj > 0 || kk > 0) ? 1u : 0u);
          }
        tc_commit(&bar[B_VFEMPTY]);
        tc_commit(&bar[B_PEMPTY + slot]);
      };
      for (int j = 0; j < nt; j++) {
        const int slot = j & 1;
        mbar_wait(&bar[B_KFFULL], j & 1, abort_flag, p.status);
        mbar_wait(&bar[B_SEMPTY + slot], ((j >> 1) & 1) ^ 1, abort_flag, p.status);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < AD / 16; kk++) {
          // A = K[128 rows, of which 64 are this tile][16 dims], B = Q^T[32 rows][16 dims]
          const uint64_t da = umma_desc_sw128(sbase + OFF_KF + (kk >> 2) * SEG + (kk & 3) * 32, 16, 1024);
          const uint64_t db = umma_desc_sw128(sbase + OFF_Q + (kk >> 2) * QSEG + (kk & 3) * 32, 16, 1024);
          tc_mma_f16(tmem + TM_S + slot * 32, da, db, IDESC_QK, kk > 0 ? 1u : 0u);
        }
        tc_commit(&bar[B_SFULL + slot]);
        tc_commit(&bar[B_KFEMPTY]);
        if (j >= 1) issue_pv(j - 1);
      }
      issue_pv(nt - 1);
      tc_commit(&bar[B_ODONE]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
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
