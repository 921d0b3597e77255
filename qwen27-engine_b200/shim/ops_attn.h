// Drop-in C++ shim: the attention operators of the reference (namespace q27, src/ops.h:50-77) with
// their exact signatures, forwarding to the q27b_attn C ABI. A non-zero status becomes the
// std::runtime_error that the reference's own implementation throws (CK() and the shape checks,
// src/common.cuh:12-13, src/attn.cu:906,929). The reference's check-and-bench tool tools/bench_attn.cu
// compiles unchanged against this directory (its "ops.h" and "common.cuh" here) and libq27b_attn.so.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/q27b_attn.h"

namespace q27 {

namespace q27b_detail {
inline void check(int rc) {
  if (rc != Q27B_OK) throw std::runtime_error(std::string(q27b_last_error()));
}
}  // namespace q27b_detail

inline size_t kv_cache_bytes(int nkvh, int n_ctx, bool q8) { return (size_t)q27b_kv_cache_bytes(nkvh, n_ctx, q8 ? 1 : 0); }

inline int attn_chunks(int nkvh) { return q27b_attn_chunks(nkvh); }

// pf / pf_bytes (an L2 prefetch hint for the next GEMV's weights) are accepted and ignored.
inline void attn_prep(const float* qg, const float* k, const float* v, const float* q_norm, const float* k_norm, float* qn,
                      void* kcache, void* vcache, const int* pos0, int T, float eps, float theta_scale, int nqh, int nkvh,
                      int n_ctx, bool q8, cudaStream_t s, const void* pf = nullptr, size_t pf_bytes = 0,
                      const int* rope3 = nullptr, const int* rdelta = nullptr) {
  (void)pf;
  (void)pf_bytes;
  q27b_detail::check(q27b_attn_prep(qg, k, v, q_norm, k_norm, qn, kcache, vcache, pos0, T, eps, theta_scale, nqh, nkvh,
                                    n_ctx, q8 ? 1 : 0, (void*)s, rope3, rdelta));
}

inline void attn_decode(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o, int8_t* xq,
                        float* xd, const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, bool q8,
                        cudaStream_t s) {
  q27b_detail::check(q27b_attn_decode(qn, qg, kcache, vcache, o, xq, xd, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8 ? 1 : 0,
                                      (void*)s));
}

inline void attn_prefill(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                         const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx, bool q8, cudaStream_t s,
                         int depth_hint = -1) {
  q27b_detail::check(q27b_attn_prefill(qn, qg, kcache, vcache, o, pos0, M, kq_scale, nqh, nkvh, n_ctx, q8 ? 1 : 0,
                                       (void*)s, depth_hint));
}

inline void attn_decode_ref(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                            const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, bool q8, cudaStream_t s) {
  q27b_detail::check(q27b_attn_decode_ref(qn, qg, kcache, vcache, o, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8 ? 1 : 0,
                                          (void*)s));
}

}  // namespace q27
