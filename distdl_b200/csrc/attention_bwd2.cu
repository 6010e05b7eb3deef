// Flash attention backward with P / dS in tensor memory (attention_bwd2_impl.cuh), built for head
// dimensions 128 and 64.
#include <cstdlib>

#include "common.cuh"
#include "runtime.cuh"

using namespace dd;

#define DD_HEAD_DIM 128
#define DD_BWD2_NS bwd2_d128
#include "attention_bwd2_impl.cuh"
#undef DD_HEAD_DIM
#undef DD_BWD2_NS

#define DD_HEAD_DIM 64
#define DD_BWD2_NS bwd2_d64
#include "attention_bwd2_impl.cuh"
#undef DD_HEAD_DIM
#undef DD_BWD2_NS

// Same contract as dd_attn_bwd for head dimensions 128 and 64, except for the scratch: `scratch`
// holds 2 * batch * Hq * S floats (delta, then the log-sum-exp in base 2).
DD_API int dd_attn_bwd2(const void* q, long long q_row, long long q_head, const void* k, long long k_row,
                        long long k_head, const void* v, long long v_row, long long v_head, const void* out,
                        const void* dout, const float* lse, float* scratch, void* dq, long long dq_row,
                        long long dq_head, void* dk, long long dk_row, long long dk_head, void* dv, long long dv_row,
                        long long dv_head, int batch, int S, int Hq, int Hkv, int Dh, int causal, float scale,
                        void* stream) {
  if (Dh == 128)
    return bwd2_d128::run(q, q_row, q_head, k, k_row, k_head, v, v_row, v_head, out, dout, lse, scratch, dq, dq_row,
                          dq_head, dk, dk_row, dk_head, dv, dv_row, dv_head, batch, S, Hq, Hkv, Dh, causal, scale, stream);
  if (Dh == 64)
    return bwd2_d64::run(q, q_row, q_head, k, k_row, k_head, v, v_row, v_head, out, dout, lse, scratch, dq, dq_row,
                         dq_head, dk, dk_row, dk_head, dv, dv_row, dv_head, batch, S, Hq, Hkv, Dh, causal, scale, stream);
  return DD_ERR_BAD_ARG;
}
