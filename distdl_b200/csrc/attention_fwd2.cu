// Two-tile flash attention forward (attention_fwd2_impl.cuh), built for head dimensions 128 and 64.
#include <cstdlib>

#include "common.cuh"
#include "runtime.cuh"

using namespace dd;

#define DD_HEAD_DIM 128
#define DD_FWD2_NS fwd2_d128
#include "attention_fwd2_impl.cuh"
#undef DD_HEAD_DIM
#undef DD_FWD2_NS

#define DD_HEAD_DIM 64
#define DD_FWD2_NS fwd2_d64
#include "attention_fwd2_impl.cuh"
#undef DD_HEAD_DIM
#undef DD_FWD2_NS

// Head dim 128 or 64, sequence length a multiple of 256.  Same argument convention as dd_attn_fwd.
DD_API int dd_attn_fwd2(const void* q, long long q_row_stride, long long q_head_stride, const void* k,
                        long long k_row_stride, long long k_head_stride, const void* v, long long v_row_stride,
                        long long v_head_stride, void* out, float* lse, int batch, int S, int Hq, int Hkv, int Dh,
                        int causal, float scale, void* stream) {
  if (Dh == 128)
    return fwd2_d128::run(q, q_row_stride, q_head_stride, k, k_row_stride, k_head_stride, v, v_row_stride,
                          v_head_stride, out, lse, batch, S, Hq, Hkv, Dh, causal, scale, stream);
  if (Dh == 64)
    return fwd2_d64::run(q, q_row_stride, q_head_stride, k, k_row_stride, k_head_stride, v, v_row_stride,
                         v_head_stride, out, lse, batch, S, Hq, Hkv, Dh, causal, scale, stream);
  return DD_ERR_BAD_ARG;
}
