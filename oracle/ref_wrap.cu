// C entry points around the reference's own attention operators (namespace q27, src/ops.h:50-77),
// so that tests and the benchmark can call the unmodified reference kernels through ctypes.
// TEST INFRASTRUCTURE ONLY: this file is compiled together with the reference's src/attn.cu and
// src/ops.cu, taken where they lie in the reference checkout, into oracle/_ref/libq27ref.so by
// oracle/build.py. Nothing of the reference is copied; nothing shipped links this.
#include "ops.h"

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>

namespace {
char g_err[512] = "";
template <class F>
int guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    std::snprintf(g_err, sizeof(g_err), "%s", e.what());
    return 1;
  }
}
}  // namespace

extern "C" {

const char* ref_last_error() { return g_err; }

uint64_t ref_kv_cache_bytes(int nkvh, int n_ctx, int q8) { return q27::kv_cache_bytes(nkvh, n_ctx, q8 != 0); }

int ref_attn_chunks(int nkvh) {
  int n = 0;
  guard([&] { n = q27::attn_chunks(nkvh); });
  return n;
}

int ref_attn_prep(const float* qg, const float* k, const float* v, const float* q_norm, const float* k_norm, float* qn,
                  void* kcache, void* vcache, const int* pos0, int T, float eps, float theta_scale, int nqh, int nkvh,
                  int n_ctx, int q8, void* stream, const int* rope3, const int* rdelta) {
  return guard([&] {
    q27::attn_prep(qg, k, v, q_norm, k_norm, qn, kcache, vcache, pos0, T, eps, theta_scale, nqh, nkvh, n_ctx, q8 != 0,
                   (cudaStream_t)stream, nullptr, 0, rope3, rdelta);
  });
}

int ref_attn_decode(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o, int8_t* xq,
                    float* xd, const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8,
                    void* stream) {
  return guard([&] {
    q27::attn_decode(qn, qg, kcache, vcache, o, xq, xd, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8 != 0,
                     (cudaStream_t)stream);
  });
}

int ref_attn_prefill(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                     const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, void* stream,
                     int depth_hint) {
  return guard([&] {
    q27::attn_prefill(qn, qg, kcache, vcache, o, pos0, M, kq_scale, nqh, nkvh, n_ctx, q8 != 0, (cudaStream_t)stream,
                      depth_hint);
  });
}

int ref_attn_decode_ref(const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                        const int* pos0, int T, float kq_scale, int nqh, int nkvh, int n_ctx, int q8, void* stream) {
  return guard([&] {
    q27::attn_decode_ref(qn, qg, kcache, vcache, o, pos0, T, kq_scale, nqh, nkvh, n_ctx, q8 != 0,
                         (cudaStream_t)stream);
  });
}

// sum_norm_q8 without an exchange (ar == nullptr, src/ops.h:101-104), for the fixture that pins the
// oracle's statement of it.
int ref_sum_norm_q8(float* x, const float* partial, int n, int rows, const float* w, float eps, float* h, int8_t* xq,
                    float* xd, void* stream) {
  return guard([&] { q27::sum_norm_q8(x, partial, n, rows, nullptr, w, eps, h, xq, xd, (cudaStream_t)stream); });
}

}  // extern "C"
