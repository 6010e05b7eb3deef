// Token routing kernels of the mixture-of-experts layers: slot assignment,
// permuted scatter into per-expert capacity buffers (optionally scaled by the
// router weight), weighted gather-sum back to token order, and the per-pair dot
// products that give the router-weight gradients.  New relative to the
// reference, whose expert layers have no router, top-k or dispatch / combine.
//
// A "pair" is one (token, choice) of the top-k routing: pair p = t * k + c has
// expert ids[p] and, after assignment, slot[p] in [0, capacity) or -1 (dropped).
#include "common.cuh"

using namespace dd;

namespace {

__global__ void moe_assign_kernel(const int* __restrict__ ids, int npairs, int E, int capacity,
                                  int* __restrict__ counters, int* __restrict__ slot) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= npairs) return;
  const int e = ids[p];
  if (e < 0 || e >= E) { slot[p] = -1; return; }
  const int s = atomicAdd(counters + e, 1);
  slot[p] = s < capacity ? s : -1;
}

// dst[e, slot, :] = (w ? w[p] : 1) * src[p / k, :]
__global__ void moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ ids,
                                        const int* __restrict__ slot, const float* __restrict__ w,
                                        __nv_bfloat16* __restrict__ dst, int npairs, int k, int capacity, int d) {
  const int dv = d >> 3;
  const long long total = (long long)npairs * dv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i / dv);
    const int c = (int)(i - (long long)p * dv) * 8;
    const int s = slot[p];
    if (s < 0) continue;
    const uint4 u = *reinterpret_cast<const uint4*>(src + (size_t)(p / k) * d + c);
    uint4 o = u;
    if (w != nullptr) {
      const float sc = w[p];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
      o.x = pack_bf16x2(a.x * sc, a.y * sc); o.y = pack_bf16x2(b.x * sc, b.y * sc);
      o.z = pack_bf16x2(cc.x * sc, cc.y * sc); o.w = pack_bf16x2(e.x * sc, e.y * sc);
    }
    *reinterpret_cast<uint4*>(dst + ((size_t)ids[p] * capacity + s) * d + c) = o;
  }
}

// dst[t, :] = sum_c (w ? w[t*k+c] : 1) * src[ids, slot, :]   (dropped pairs contribute 0)
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ ids,
                                       const int* __restrict__ slot, const float* __restrict__ w,
                                       __nv_bfloat16* __restrict__ dst, int tokens, int k, int capacity, int d) {
  const int dv = d >> 3;
  const long long total = (long long)tokens * dv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / dv);
    const int c = (int)(i - (long long)t * dv) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int p = t * k + j;
      const int s = slot[p];
      if (s < 0) continue;
      const float sc = w ? w[p] : 1.f;
      const uint4 u = *reinterpret_cast<const uint4*>(src + ((size_t)ids[p] * capacity + s) * d + c);
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
      acc[0] += sc * a.x; acc[1] += sc * a.y; acc[2] += sc * b.x; acc[3] += sc * b.y;
      acc[4] += sc * cc.x; acc[5] += sc * cc.y; acc[6] += sc * e.x; acc[7] += sc * e.y;
    }
    uint4 o = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                         pack_bf16x2(acc[6], acc[7]));
    *reinterpret_cast<uint4*>(dst + (size_t)t * d + c) = o;
  }
}

// out[p] = <a[p / k, :], b[ids[p], slot[p], :]>   (0 for dropped pairs); one warp per pair
__global__ void moe_pair_dot_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                    const int* __restrict__ ids, const int* __restrict__ slot,
                                    float* __restrict__ out, int npairs, int k, int capacity, int d) {
  const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= npairs) return;
  const int lane = threadIdx.x & 31;
  const int s = slot[p];
  float acc = 0.f;
  if (s >= 0) {
    const __nv_bfloat16* ar = a + (size_t)(p / k) * d;
    const __nv_bfloat16* br = b + ((size_t)ids[p] * capacity + s) * d;
    for (int c = lane * 8; c < d; c += 256) {
      const uint4 u = *reinterpret_cast<const uint4*>(ar + c);
      const uint4 v = *reinterpret_cast<const uint4*>(br + c);
      float2 x, y;
      x = unpack_bf16x2(u.x); y = unpack_bf16x2(v.x); acc += x.x * y.x + x.y * y.y;
      x = unpack_bf16x2(u.y); y = unpack_bf16x2(v.y); acc += x.x * y.x + x.y * y.y;
      x = unpack_bf16x2(u.z); y = unpack_bf16x2(v.z); acc += x.x * y.x + x.y * y.y;
      x = unpack_bf16x2(u.w); y = unpack_bf16x2(v.w); acc += x.x * y.x + x.y * y.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[p] = acc;
}

inline int grid_for(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  if (b > 148 * 16) b = 148 * 16;
  return (int)(b < 1 ? 1 : b);
}
}  // namespace

#define S(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<__nv_bfloat16*>(p)
#define CBF(p) reinterpret_cast<const __nv_bfloat16*>(p)

// counters[E] must be zero on entry.
DD_API int dd_moe_assign(const int* ids, int npairs, int E, int capacity, int* counters, int* slot, void* stream) {
  if (npairs <= 0) return DD_OK;
  moe_assign_kernel<<<(npairs + 255) / 256, 256, 0, S(stream)>>>(ids, npairs, E, capacity, counters, slot);
  return (int)cudaGetLastError();
}
DD_API int dd_moe_scatter_rows(const void* src, const int* ids, const int* slot, const float* w, void* dst,
                               int npairs, int k, int capacity, int d, void* stream) {
  if (d % 8) return DD_ERR_BAD_ARG;
  if (npairs <= 0) return DD_OK;
  moe_scatter_rows_kernel<<<grid_for((long long)npairs * (d / 8), 256), 256, 0, S(stream)>>>(
      CBF(src), ids, slot, w, BF(dst), npairs, k, capacity, d);
  return (int)cudaGetLastError();
}
DD_API int dd_moe_gather_rows(const void* src, const int* ids, const int* slot, const float* w, void* dst,
                              int tokens, int k, int capacity, int d, void* stream) {
  if (d % 8) return DD_ERR_BAD_ARG;
  if (tokens <= 0) return DD_OK;
  moe_gather_rows_kernel<<<grid_for((long long)tokens * (d / 8), 256), 256, 0, S(stream)>>>(
      CBF(src), ids, slot, w, BF(dst), tokens, k, capacity, d);
  return (int)cudaGetLastError();
}
DD_API int dd_moe_pair_dot(const void* a, const void* b, const int* ids, const int* slot, float* out, int npairs,
                           int k, int capacity, int d, void* stream) {
  if (d % 8) return DD_ERR_BAD_ARG;
  if (npairs <= 0) return DD_OK;
  moe_pair_dot_kernel<<<(npairs + 7) / 8, 256, 0, S(stream)>>>(CBF(a), CBF(b), ids, slot, out, npairs, k, capacity, d);
  return (int)cudaGetLastError();
}
