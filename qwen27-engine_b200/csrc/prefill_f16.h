// Launcher of the f16-cache prefill kernel (prefill_f16.cu), called by q27b_attn_prefill* when the
// cache is f16.
#pragma once
#include "host.h"

#include <algorithm>
#include <cstdlib>

namespace q27b {

// How the CTAs of a prefill call (one per 128-token query tile and head, one CTA per SM at a time)
// split their positions. Tiles [0, ts) are split ns ways (partials + merge), tiles >= ts are not.
//  * Few CTAs: every tile is split, enough CTAs for every SM and at least 2048 positions per split
//    (the reference's rule, src/attn.cu:945-951). Q27_ATTN_SPLIT forces this form (src/attn.cu:952).
//  * More CTAs than SMs on a deep prefix (all CTAs about equally long): the CTAs beyond the last full
//    wave would leave most SMs idle for a whole CTA time (384 CTAs on 148 SMs: 3 rounds for 2.6
//    rounds of work). The unsplit CTAs are launched first and only the earliest ts tiles - as many
//    CTAs as the remainder - are cut into ns pieces that fill the machine evenly at the end; ns is
//    the count that minimises the modelled makespan. Only ts / tiles of the rows pay for a merge.
struct SplitPlan {
  int ts, ns;
};
inline SplitPlan plan_prefill_split(int tiles, int nqh, int n_sm, int M, int depth_hint, bool must_merge) {
  const int ctas = tiles * nqh;
  int ns = 1;
  const int ns_max = depth_hint >= 0 ? std::max(1, std::min(8, (depth_hint + M) / 2048)) : 1;
  if (depth_hint >= 0) ns = std::max(1, std::min((2 * n_sm + ctas - 1) / ctas, ns_max));
  if (const char* e = getenv("Q27_ATTN_SPLIT")) {
    const int f = atoi(e);
    if (f > 0) return {f > 1 || must_merge ? tiles : 0, std::max(std::min(f, 64), must_merge ? 2 : 1)};
  }
  if (must_merge) return {tiles, std::max(ns, 2)};
  if (ns > 1) return {tiles, ns};
  const char* tail = getenv("Q27B_PREFILL_TAIL_SPLIT");
  if ((tail && tail[0] == '0') || depth_hint < 4 * M || ctas <= n_sm || ctas % n_sm == 0 || ns_max < 2) return {0, 1};
  const int ts = std::min(tiles, (ctas % n_sm + nqh - 1) / nqh);
  const int U = ctas - ts * nqh, a = U / n_sm, b = U % n_sm;
  double best = (double)((ctas + n_sm - 1) / n_sm);  // not splitting at all
  int best_ns = 1;
  for (int k = 2; k <= ns_max; k++) {
    const long P = (long)ts * nqh * k, cap = b ? (long)(n_sm - b) * k : 0;
    double t = a + (b ? 1.0 : 0.0);
    if (P > cap) t += (double)((P - cap + n_sm - 1) / n_sm) / k;
    t += k * 1400.0 / (depth_hint + M);  // per piece: Q tile, pipeline fill, partials, merge (measured at 32k and 148k)
    if (t < best) best = t, best_ns = k;
  }
  if (tail && atoi(tail) > 1) best_ns = std::min(atoi(tail), ns_max);  // tuning: Q27B_PREFILL_TAIL_SPLIT=<pieces>
  return best_ns > 1 ? SplitPlan{ts, best_ns} : SplitPlan{0, 1};
}

// The f16-QK kernel: on an f16 cache (q8 = false), or on a q8_0 cache whose K and V it dequantises to
// f16 on the way (q8 = true; the reference's Q27_ATTN_I8=0 path). o (f32) or xq/xd (q8_1, written by
// the merge kernel of the split path). Same contract as q27b_attn_prefill.
int launch_prefill_f16(DeviceCtx* ctx, const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                       int8_t* xq, float* xd, const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx, bool q8,
                       int depth_hint, cudaStream_t s);

}  // namespace q27b
