// Shared device helpers of the sm_100a attention kernels: PTX wrappers (mbarrier, TMA, tcgen05,
// warp MMA), bounded waits, and the constants of the cache layout (reference src/ops.h:50-53).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace q27b {

constexpr int AD = 256;          // head dim (reference src/attn.cu:22)
constexpr int GQA = 6;           // query heads per KV head (src/attn.cu:23)
constexpr int MAXR = GQA * 4;    // query rows per KV head in a decode call (src/attn.cu:27)
constexpr int PROW = AD + 2;     // floats per partial row: m, l, O[256] (src/attn.cu:26)
constexpr float M_INIT = -1e30f; // finite start of the running max (src/attn.cu:28)
constexpr float LOG2E = 1.4426950408889634f;

// Bits of the per-device status word written by kernels.
constexpr int ST_WAIT_EXPIRED = 1;   // a bounded mbarrier wait gave up
constexpr int ST_BAD_PAGE = 2;       // a page-table entry was out of range (the page was skipped)

// The reference's kernels all start with these two (src/common.cuh:17-21), so that they stay
// legal under its programmatic-dependent launches.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint64_t* bar, uint32_t n) {  // n arrivals at once
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Same with a suspend-time hint (ns): the thread may sleep in hardware until the phase completes
// or the time is up, instead of polling and taking issue slots from the working warps.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait. `abort_flag` lives in shared memory: once any thread of the CTA has given up,
// every later wait returns at once, so the CTA drains to its end instead of hanging. The first
// thread to give up records ST_WAIT_EXPIRED in the global status word. Results of such a CTA
// are garbage; the host reports the status.
//
// The polling loop is deliberately NOT inlined: these kernels run several differently specialised
// warps per scheduler, their code is tens of kilobytes, and they are sensitive to instruction-cache
// pressure (measured on the prefill kernel: +40 % throughput from moving this loop out of line at
// its ~50 call sites). The inlined part is one try_wait, which is all that a wait on a barrier that
// has already completed costs.
constexpr long long WAIT_LIMIT_NS = 2000000000ll;  // two seconds ...
constexpr uint32_t WAIT_MIN_POLLS = 1u << 20;      // ... and at least this many polls (a jump of the timer alone never ends a wait)
constexpr uint32_t WAIT_HINT_NS = 1000u;
#ifdef Q27B_INLINE_WAITS  // a kernel whose warps all run the same code may prefer the loop inline
#define Q27B_WAIT_SLOW_ATTR __forceinline__
#else
#define Q27B_WAIT_SLOW_ATTR __noinline__
#endif
static __device__ Q27B_WAIT_SLOW_ATTR void mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  unsigned long long t0 = 0;
  for (uint32_t i = 1;; i++) {
    if (mbar_try_wait_hint(bar, parity, WAIT_HINT_NS)) return;
    if ((i & 255u) == 0) {
      if (*abort_flag) return;
      const unsigned long long t = global_ns();
      if (t0 == 0) t0 = t;
      else if (i >= WAIT_MIN_POLLS && (long long)(t - t0) > WAIT_LIMIT_NS) break;
    }
  }
  *abort_flag = 1;
  if (status) atomicOr(status, ST_WAIT_EXPIRED);
}
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (mbar_try_wait(bar, parity)) return;
  mbar_wait_slow(bar, parity, abort_flag, status);
}

// The same for a wait that is expected to be long while other warps of the scheduler have work: between
// polls the warp sleeps, so that it is not eligible and takes no issue slots (a polling warp is always
// eligible). Costs up to the sleep time in latency.
static __device__ __forceinline__ void mbar_wait_sleeping(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                          uint32_t sleep_ns = 200) {
  if (mbar_try_wait(bar, parity)) return;
  unsigned long long t0 = 0;
  for (uint32_t i = 1;; i++) {
    __nanosleep(sleep_ns);
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 63u) == 0) {
      if (*abort_flag) return;
      const unsigned long long t = global_ns();
      if (t0 == 0) t0 = t;
      else if (i >= (1u << 16) && (long long)(t - t0) > WAIT_LIMIT_NS) break;
    }
  }
  *abort_flag = 1;
  if (status) atomicOr(status, ST_WAIT_EXPIRED);
}

// ---- exchange over peer memory: every float travels as one 8-byte word {value, tag}, tag = the step it belongs
// to (epoch + 1). An aligned 8-byte store is one transaction, so a reader that finds the tag of the current
// step has the value of the current step: no fence and no separate flag are needed (a system-scope fence, which
// the flag form needs between the rows and the flag, was measured at 10 us and more per kernel on this GPU).
__device__ __forceinline__ void ll_store(uint64_t* p, float v, int tag) {
  const uint64_t w = ((uint64_t)(uint32_t)tag << 32) | (uint64_t)__float_as_uint(v);
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
// Waits (bounded: about a second with the sleeps, then ok = false) for the word to carry `tag`.
__device__ __forceinline__ float ll_load(const uint64_t* p, int tag, bool& ok) {
  for (uint32_t i = 0; i < (1u << 22); i++) {
    uint64_t w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    if ((int)(uint32_t)(w >> 32) == tag) return __uint_as_float((uint32_t)w);
    if (i > 64) __nanosleep(200);
  }
  ok = false;
  return 0.f;
}

// After a wait has given up, a CTA drains to its end without synchronisation. Before it frees
// tensor memory and exits it gives the copies and MMAs that it issued earlier time to land
// (microseconds of work; this sleeps 100 us), so that nothing is still writing into shared or
// tensor memory that the next CTA on this SM will own.
__device__ __forceinline__ void drain_after_abort(volatile int* abort_flag) {
  if (*abort_flag)
    for (int i = 0; i < 100; i++) __nanosleep(1000);
}

// ------------------------------------------------------------------ TMA (plain per-CTA loads only)
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// The same box into L2 only: a later tma_load_2d of it then costs an L2 hit instead of the DRAM latency.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Byte offset of 16-byte chunk `chunk` (0..7) of 128-byte row `row` in a tile stored with the
// 128-byte TMA / UMMA swizzle (tile base 1024-byte aligned): chunk index XOR (row mod 8).
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }

// ------------------------------------------------------------------ warp MMA (legacy tensor path)
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *(const uint32_t*)&h;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *(const uint32_t*)&h; }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *(const __half2*)&u; }

// Two int8 values (already XORed with 0x80, sitting in the low bytes of the two f16 lanes of
// `biased` = 0x64xx64xx, i.e. 1024 + q + 128 each) times a pair of f16 scales: (x - 1152) is the
// exact integer, the product is rounded once to f16. Same value as the reference's dequantisation
// (cvt_q8_16, src/attn.cu:59-76; cache_val, src/attn.cu:827-832).
__device__ __forceinline__ uint32_t dq_pair(uint32_t biased, __half2 scale) {
  const __half2 off = __half2half2(__ushort_as_half((unsigned short)0x6480));  // 1152.0
  return h2_as_u32(__hmul2(__hsub2(u32_as_h2(biased), off), scale));
}

// ------------------------------------------------------------------ packed f32x2 arithmetic (sm_100)
// Two f32 values in one 64-bit register pair; one instruction does both lanes.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// ------------------------------------------------------------------ tcgen05 (5th-gen tensor cores, TMEM)
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrives on `bar` when every tcgen05.mma issued by this thread so far has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by one thread.
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}

// Same with the A operand in tensor memory (lane = row, two f16 per 32-bit column along K).
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accum)
      : "memory");
}

// Shared-memory matrix descriptor of tcgen05.mma (64 bit): start address >> 4 in bits 0-13,
// leading byte offset >> 4 in 16-29, stride byte offset >> 4 in 32-45, descriptor version 1 in
// 46-47, swizzle mode in 61-63 (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor of tcgen05.mma kind::f16 / kind::i8 (32 bit): D format in bits 4-5
// (0 f16, 1 f32, 2 s32), A format in 7-9 and B format in 10-12 (f16: 0 = f16; i8: 1 = signed),
// A / B major in 15 / 16 (0 = K-major, 1 = MN-major), N >> 3 in 17-22, M >> 4 in 24-28.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t c_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t a_mn_major,
                                                  uint32_t b_mn_major, uint32_t M, uint32_t N) {
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((N >> 3) << 17) |
         ((M >> 4) << 24);
}

// 32 lanes x 32 columns of 32-bit TMEM cells -> 32 registers per thread (thread = lane).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}

}  // namespace q27b
