// Launcher of the f16-cache prefill kernel (prefill_f16.cu), called by q27b_attn_prefill* when the
// cache is f16.
#pragma once
#include "host.h"

namespace q27b {

// o (f32) or xq/xd (q8_1, written by the merge kernel of the split path). Same contract as the q8_0
// path of q27b_attn_prefill.
int launch_prefill_f16(DeviceCtx* ctx, const float* qn, const float* qg, const void* kcache, const void* vcache, float* o,
                       int8_t* xq, float* xd, const int* pos0, int M, float kq_scale, int nqh, int nkvh, int n_ctx,
                       int depth_hint, cudaStream_t s);

}  // namespace q27b
