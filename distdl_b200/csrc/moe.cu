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

// Slots are positions in the arrival order of the pairs at their expert, and the arrival order is
// the pair index: the result does not depend on how the threads are scheduled, so the same pairs
// are dropped at an overflowing expert in every run.  Two steps over chunks of kChunk tokens (one
// CTA each, one thread per token, k pairs per thread):
//   histogram: hist[chunk][e] = pairs of the chunk routed to e
//   slots    : base[e] = sum of the earlier chunks' histograms; inside the chunk a pair's rank is the
//              number of earlier lanes (and warps) of the CTA with a pair for the same expert.
constexpr int kChunk = 256;
constexpr int kMaxExperts = 64;

__global__ void __launch_bounds__(kChunk)
moe_hist_kernel(const int* __restrict__ ids, int tokens, int k, int E, int* __restrict__ hist) {
  __shared__ int s_hist[kMaxExperts];
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  const int t = blockIdx.x * kChunk + threadIdx.x;
  if (t < tokens)
    for (int c = 0; c < k; ++c) {
      const int e = ids[(size_t)t * k + c];
      if (e >= 0 && e < E) atomicAdd(&s_hist[e], 1);
    }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[(size_t)blockIdx.x * E + e] = s_hist[e];
}

// The k experts of one token must differ (top-k routing) or k must be 1.
__global__ void __launch_bounds__(kChunk)
moe_slot_kernel(const int* __restrict__ ids, int tokens, int k, int E, int capacity, const int* __restrict__ hist,
                int* __restrict__ totals, int* __restrict__ slot) {
  __shared__ unsigned s_mask[kChunk / 32][kMaxExperts];     // lanes of a warp with a pair for expert e
  __shared__ int s_base[kChunk / 32][kMaxExperts];          // pairs for e before this warp
  for (int i = threadIdx.x; i < (kChunk / 32) * kMaxExperts; i += blockDim.x) (&s_mask[0][0])[i] = 0u;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kChunk + threadIdx.x;
  if (t < tokens)
    for (int c = 0; c < k; ++c) {
      const int e = ids[(size_t)t * k + c];
      if (e >= 0 && e < E) atomicOr(&s_mask[warp][e], 1u << lane);
    }
  __syncthreads();
  if ((int)threadIdx.x < E) {
    const int e = threadIdx.x;
    int run = 0;
    for (int cta = 0; cta < (int)blockIdx.x; ++cta) run += hist[(size_t)cta * E + e];
    for (int w = 0; w < kChunk / 32; ++w) { s_base[w][e] = run; run += __popc(s_mask[w][e]); }
    if (blockIdx.x == gridDim.x - 1) totals[e] = run;
  }
  __syncthreads();
  if (t < tokens)
    for (int c = 0; c < k; ++c) {
      const int e = ids[(size_t)t * k + c];
      int sl = -1;
      if (e >= 0 && e < E) {
        sl = s_base[warp][e] + __popc(s_mask[warp][e] & ((1u << lane) - 1u));
        if (sl >= capacity) sl = -1;
      }
      slot[(size_t)t * k + c] = sl;
    }
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

// ---------------------------------------------------------------------------
// Router: softmax over the experts, top-k, renormalised weights, the chunk's expert
// histogram and the column sums of the probabilities (for the load-balancing loss) in one
// kernel; one thread per token, the E (<= EMAX) logits of a token in registers.
//   p = softmax(l);  S = top-k of p;  w_i = p_i / sum_{j in S} p_j  (i in S)
// Outputs per pair (t, c): ids, w; hist[chunk][e] for moe_slot_kernel, which follows and
// turns the histograms into slots (arrival order at the expert = pair index order, -1 beyond
// the capacity).  prob_sum[e] ends as sum_t p[t, e] and must be zero on entry.
// ---------------------------------------------------------------------------
template <int EMAX>
__global__ void __launch_bounds__(256)
moe_router_fwd_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int tokens, int E, int k, int capacity,
                      int* __restrict__ ids, float* __restrict__ w, int* __restrict__ hist,
                      float* __restrict__ prob_sum) {
  __shared__ float s_sum[EMAX];
  __shared__ int s_hist[EMAX];
  for (int e = threadIdx.x; e < EMAX; e += blockDim.x) { s_sum[e] = 0.f; s_hist[e] = 0; }
  __syncthreads();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < tokens) {
    float p[EMAX];
    float m = -INFINITY;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      p[e] = e < E ? __bfloat162float(logits[(size_t)t * ld + e]) : -INFINITY;
      m = fmaxf(m, p[e]);
    }
    float z = 0.f;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) { p[e] = e < E ? __expf(p[e] - m) : 0.f; z += p[e]; }
    const float inv = 1.f / z;
#pragma unroll
    for (int e = 0; e < EMAX; ++e) {
      p[e] *= inv;
      if (e < E) atomicAdd(&s_sum[e], p[e]);
    }
    unsigned long long taken = 0ull;
    float wsel[8];
    int isel[8];
    float zs = 0.f;
    for (int c = 0; c < k; ++c) {
      float best = -1.f;
      int bi = 0;
#pragma unroll
      for (int e = 0; e < EMAX; ++e)
        if (e < E && !((taken >> e) & 1ull) && p[e] > best) { best = p[e]; bi = e; }
      taken |= 1ull << bi;
      wsel[c] = best; isel[c] = bi; zs += best;
    }
    const float invs = 1.f / zs;
    for (int c = 0; c < k; ++c) {
      const int pr = t * k + c;
      ids[pr] = isel[c];
      w[pr] = wsel[c] * invs;
      atomicAdd(&s_hist[isel[c]], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (s_sum[e] != 0.f) atomicAdd(prob_sum + e, s_sum[e]);
    hist[(size_t)blockIdx.x * E + e] = s_hist[e];
  }
}

// dl_i = p_i (c_i - sum_e c_e p_e)  +  [i in S] w_i (dw_i - sum_{j in S} w_j dw_j)
// with c = gradient arriving on prob_sum and dw on the pair weights; columns >= E get 0.
template <int EMAX>
__global__ void __launch_bounds__(256)
moe_router_bwd_kernel(const __nv_bfloat16* __restrict__ logits, int ld, int tokens, int E, int k,
                      const int* __restrict__ ids, const float* __restrict__ w, const float* __restrict__ dw,
                      const float* __restrict__ coef, __nv_bfloat16* __restrict__ dlogits) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  float p[EMAX];
  float m = -INFINITY;
#pragma unroll
  for (int e = 0; e < EMAX; ++e) {
    p[e] = e < E ? __bfloat162float(logits[(size_t)t * ld + e]) : -INFINITY;
    m = fmaxf(m, p[e]);
  }
  float z = 0.f;
#pragma unroll
  for (int e = 0; e < EMAX; ++e) { p[e] = e < E ? __expf(p[e] - m) : 0.f; z += p[e]; }
  const float inv = 1.f / z;
  float cp = 0.f;
#pragma unroll
  for (int e = 0; e < EMAX; ++e) {
    p[e] *= inv;
    if (e < E && coef != nullptr) cp += coef[e] * p[e];
  }
  float g[EMAX];
#pragma unroll
  for (int e = 0; e < EMAX; ++e) g[e] = (e < E && coef != nullptr) ? p[e] * (coef[e] - cp) : 0.f;
  if (dw != nullptr) {
    float wd = 0.f;
    for (int c = 0; c < k; ++c) wd += w[t * k + c] * dw[t * k + c];
    for (int c = 0; c < k; ++c) {
      const int i = ids[t * k + c];
      const float add = w[t * k + c] * (dw[t * k + c] - wd);
#pragma unroll
      for (int e = 0; e < EMAX; ++e)
        if (e == i) g[e] += add;
    }
  }
  for (int e = 0; e < ld; ++e) {
    float v = 0.f;
#pragma unroll
    for (int q = 0; q < EMAX; ++q)
      if (q == e) v = g[q];
    dlogits[(size_t)t * ld + e] = __float2bfloat16(v);
  }
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
// counters: (chunks + 1) * E ints with chunks = dd_moe_chunks(npairs): [0, E) receives the number
// of pairs per expert, the rest is scratch (nothing has to be zero on entry).  E <= 64.
DD_API int dd_moe_chunks(int tokens) { return (tokens + kChunk - 1) / kChunk; }
DD_API int dd_moe_assign(const int* ids, int npairs, int E, int capacity, int* counters, int* slot, void* stream) {
  if (E < 1 || E > kMaxExperts) return DD_ERR_BAD_ARG;
  if (npairs <= 0) return DD_OK;
  const int grid = dd_moe_chunks(npairs);
  moe_hist_kernel<<<grid, kChunk, 0, S(stream)>>>(ids, npairs, 1, E, counters + E);
  moe_slot_kernel<<<grid, kChunk, 0, S(stream)>>>(ids, npairs, 1, E, capacity, counters + E, counters, slot);
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

// logits [tokens, ld] bf16 (columns >= E are padding); E <= 64, k <= 8, k <= E.  counters as for
// dd_moe_assign with chunks = dd_moe_chunks(tokens); prob_sum [E] must be zero on entry.
DD_API int dd_moe_router_fwd(const void* logits, int ld, int tokens, int E, int k, int capacity, int* ids, float* w,
                             int* slot, int* counters, float* prob_sum, void* stream) {
  if (E < 1 || E > kMaxExperts || k < 1 || k > 8 || k > E || ld < E) return DD_ERR_BAD_ARG;
  if (tokens <= 0) return DD_OK;
  static_assert(kChunk == 256, "the router kernel handles one chunk of 256 tokens per CTA");
  const int grid = dd_moe_chunks(tokens);
  int* hist = counters + E;
  if (E <= 8)
    moe_router_fwd_kernel<8><<<grid, 256, 0, S(stream)>>>(CBF(logits), ld, tokens, E, k, capacity, ids, w, hist, prob_sum);
  else if (E <= 16)
    moe_router_fwd_kernel<16><<<grid, 256, 0, S(stream)>>>(CBF(logits), ld, tokens, E, k, capacity, ids, w, hist, prob_sum);
  else if (E <= 32)
    moe_router_fwd_kernel<32><<<grid, 256, 0, S(stream)>>>(CBF(logits), ld, tokens, E, k, capacity, ids, w, hist, prob_sum);
  else
    moe_router_fwd_kernel<64><<<grid, 256, 0, S(stream)>>>(CBF(logits), ld, tokens, E, k, capacity, ids, w, hist, prob_sum);
  moe_slot_kernel<<<grid, kChunk, 0, S(stream)>>>(ids, tokens, k, E, capacity, hist, counters, slot);
  return (int)cudaGetLastError();
}
// dw [tokens * k] and coef [E] may each be null (no gradient from that output).
DD_API int dd_moe_router_bwd(const void* logits, int ld, int tokens, int E, int k, const int* ids, const float* w,
                             const float* dw, const float* coef, void* dlogits, void* stream) {
  if (E < 1 || E > 64 || k < 1 || k > 8 || ld < E) return DD_ERR_BAD_ARG;
  if (tokens <= 0) return DD_OK;
  const int grid = (tokens + 255) / 256;
  if (E <= 8)
    moe_router_bwd_kernel<8><<<grid, 256, 0, S(stream)>>>(CBF(logits), ld, tokens, E, k, ids, w, dw, coef, BF(dlogits));
  else if (E <= 16)
    moe_router_bwd_kernel<16><<<grid, 256, 0, S(stream)>>>(CBF(logits), ld, tokens, E, k, ids, w, dw, coef, BF(dlogits));
  else if (E <= 32)
    moe_router_bwd_kernel<32><<<grid, 256, 0, S(stream)>>>(CBF(logits), ld, tokens, E, k, ids, w, dw, coef, BF(dlogits));
  else
    moe_router_bwd_kernel<64><<<grid, 256, 0, S(stream)>>>(CBF(logits), ld, tokens, E, k, ids, w, dw, coef, BF(dlogits));
  return (int)cudaGetLastError();
}
