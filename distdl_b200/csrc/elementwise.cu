// Memory-bound sm_100a kernels: RMSNorm / LayerNorm (forward, backward),
// SwiGLU and GELU (forward, backward), rotary embedding, embedding gather and
// scatter-add, fused softmax-cross-entropy, fused AdamW on fp32 master weights,
// sum of squares, residual add, cast.  All of them move 16 bytes per thread per
// access and accumulate in fp32.
#include <cstdio>

#include "common.cuh"
#include "no_alloc.h"

using namespace dd;

namespace {

constexpr int kNormThreads = 256;
constexpr int kMaxVec = 4;  // 8-element vectors per thread: rows of up to 8192 elements

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (blockDim.x >> 5)) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ---------------------------------------------------------------------------
// Norm kernels.  A CTA of 256 threads works on R rows at a time; thread t owns the
// 8-element vectors t, t + 256, ... (VEC of them, so rows of up to VEC * 2048
// elements) of every row.  All loads of the R rows are issued before the first
// use, and one block reduction serves the R rows, so the bytes in flight per SM
// (what a memory-bound kernel lives on) do not depend on a single row's round trip.
// Rows are kept as packed bf16 in registers and unpacked where needed: VEC and R
// are template parameters so that the register count follows the row length.
// ---------------------------------------------------------------------------
constexpr int kNormWarps = kNormThreads / 32;

// Sums of R values over the CTA at once; red: kNormWarps * R floats of shared memory.
template <int R>
__device__ __forceinline__ void block_sum_n(float (&v)[R], float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int r = 0; r < R; ++r) v[r] = warp_sum(v[r]);
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r) red[warp * R + r] = v[r];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < kNormWarps; ++w) t += red[w * R + r];
    v[r] = t;
  }
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// Norm forward.  RMS: y = x * rstd * w (+b).  LayerNorm: y = (x-mean)*rstd*w + b.
// stats[row] = {mean, rstd} (mean = 0 for RMS).  Optional residual: x + res is written
// to xsum first and the (rounded) sum is what gets normalised.
template <bool RMS, int VEC, int R>
__global__ void __launch_bounds__(kNormThreads)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                __nv_bfloat16* __restrict__ xsum, const __nv_bfloat16* __restrict__ w,
                const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, float2* __restrict__ stats,
                int rows, int d, float eps) {
  __shared__ float red[kNormWarps * R];
  const int nvec = d >> 3;
  const float inv_d = 1.f / (float)d;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R) {
    uint4 v[R][VEC];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int vi = threadIdx.x + i * kNormThreads;
        v[r][i] = make_uint4(0, 0, 0, 0);
        if (vi < nvec && row0 + r < rows)
          v[r][i] = *reinterpret_cast<const uint4*>(x + (size_t)(row0 + r) * d + vi * 8);
      }
    if (res != nullptr) {
      uint4 q[R][VEC];
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const int vi = threadIdx.x + i * kNormThreads;
          q[r][i] = make_uint4(0, 0, 0, 0);
          if (vi < nvec && row0 + r < rows)
            q[r][i] = *reinterpret_cast<const uint4*>(res + (size_t)(row0 + r) * d + vi * 8);
        }
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const int vi = threadIdx.x + i * kNormThreads;
          float a[8], c[8];
          unpack8(v[r][i], a);
          unpack8(q[r][i], c);
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] += c[j];
          v[r][i] = pack8(a);                   // normalise exactly what is stored
          if (xsum != nullptr && vi < nvec && row0 + r < rows)
            *reinterpret_cast<uint4*>(xsum + (size_t)(row0 + r) * d + vi * 8) = v[r][i];
        }
    }
    float s[R], ss[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      s[r] = 0.f; ss[r] = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        float a[8];
        unpack8(v[r][i], a);
#pragma unroll
        for (int j = 0; j < 8; ++j) { s[r] += a[j]; ss[r] += a[j] * a[j]; }
      }
    }
    float mean[R], rstd[R];
    if (RMS) {
      block_sum_n<R>(ss, red);
#pragma unroll
      for (int r = 0; r < R; ++r) { mean[r] = 0.f; rstd[r] = rsqrtf(ss[r] * inv_d + eps); }
    } else {
      block_sum_n<R>(s, red);
      float sq[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        mean[r] = s[r] * inv_d;
        sq[r] = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const int vi = threadIdx.x + i * kNormThreads;
          if (vi < nvec) {
            float a[8];
            unpack8(v[r][i], a);
#pragma unroll
            for (int j = 0; j < 8; ++j) { const float t = a[j] - mean[r]; sq[r] += t * t; }
          }
        }
      }
      block_sum_n<R>(sq, red);
#pragma unroll
      for (int r = 0; r < R; ++r) rstd[r] = rsqrtf(sq[r] * inv_d + eps);
    }
    if (threadIdx.x < R && stats != nullptr && row0 + threadIdx.x < rows) {
#pragma unroll
      for (int r = 0; r < R; ++r)
        if (r == (int)threadIdx.x) stats[row0 + r] = make_float2(mean[r], rstd[r]);
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int vi = threadIdx.x + i * kNormThreads;
      if (vi < nvec) {
        float wv[8], bv[8];
        if (w != nullptr) load8(w + vi * 8, wv);
        else {
#pragma unroll
          for (int j = 0; j < 8; ++j) wv[j] = 1.f;
        }
        if (b != nullptr) load8(b + vi * 8, bv);
        else {
#pragma unroll
          for (int j = 0; j < 8; ++j) bv[j] = 0.f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (row0 + r < rows) {
            float a[8], o[8];
            unpack8(v[r][i], a);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = (a[j] - mean[r]) * rstd[r] * wv[j] + bv[j];
            store8(y + (size_t)(row0 + r) * d + vi * 8, o);
          }
        }
      }
    }
  }
}

// Norm backward.  g = dy*w, xh = (x-mean)*rstd:
//   RMS: dx = rstd*(g - xh*mean(g*xh));  LN: dx = rstd*(g - mean(g) - xh*mean(g*xh))
// dw/db partial sums per CTA go to `partial` ([gridDim.x][2][d] fp32, a scratch
// buffer); norm_bwd_reduce_kernel folds them.  dx may alias dy.  WANT_DB: the
// second half of a CTA's slice (db) is only accumulated and written when asked for.
// If dres_in is given, it is added to dx (gradient of the residual stream).
template <bool RMS, int VEC, int R, bool WANT_DB>
__global__ void __launch_bounds__(kNormThreads)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const float2* __restrict__ stats,
                const __nv_bfloat16* __restrict__ dres_in, __nv_bfloat16* __restrict__ dx,
                float* __restrict__ partial, int rows, int d) {
  __shared__ float red[kNormWarps * R];
  const int nvec = d >> 3;
  const float inv_d = 1.f / (float)d;
  float dw[VEC][8], db[WANT_DB ? VEC : 1][8];
#pragma unroll
  for (int i = 0; i < VEC; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) { dw[i][j] = 0.f; if (WANT_DB) db[i][j] = 0.f; }
  float wv[VEC][8];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int vi = threadIdx.x + i * kNormThreads;
    if (w != nullptr && vi < nvec) load8(w + vi * 8, wv[i]);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[i][j] = 1.f;
    }
  }
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R) {
    uint4 pdy[R][VEC], px[R][VEC];
    float mean[R], rstd[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool live = row0 + r < rows;
      const float2 st = live ? stats[row0 + r] : make_float2(0.f, 0.f);
      mean[r] = st.x; rstd[r] = st.y;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int vi = threadIdx.x + i * kNormThreads;
        pdy[r][i] = make_uint4(0, 0, 0, 0);
        px[r][i] = make_uint4(0, 0, 0, 0);
        if (live && vi < nvec) {
          pdy[r][i] = *reinterpret_cast<const uint4*>(dy + (size_t)(row0 + r) * d + vi * 8);
          px[r][i] = *reinterpret_cast<const uint4*>(x + (size_t)(row0 + r) * d + vi * 8);
        }
      }
    }
    float sg[R], sgx[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      sg[r] = 0.f; sgx[r] = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int vi = threadIdx.x + i * kNormThreads;
        if (vi < nvec) {
          float dyv[8], xv[8];
          unpack8(pdy[r][i], dyv);
          unpack8(px[r][i], xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xh = (xv[j] - mean[r]) * rstd[r];
            const float g = dyv[j] * wv[i][j];
            dw[i][j] += dyv[j] * xh;
            if (WANT_DB) db[i][j] += dyv[j];
            sg[r] += g;
            sgx[r] += g * xh;
          }
        }
      }
    }
    block_sum_n<R>(sgx, red);
    if (!RMS) block_sum_n<R>(sg, red);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (row0 + r >= rows) continue;
      const float mgx = sgx[r] * inv_d, mg = RMS ? 0.f : sg[r] * inv_d;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int vi = threadIdx.x + i * kNormThreads;
        if (vi < nvec) {
          float dyv[8], xv[8], o[8];
          unpack8(pdy[r][i], dyv);
          unpack8(px[r][i], xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float xh = (xv[j] - mean[r]) * rstd[r];
            o[j] = rstd[r] * (dyv[j] * wv[i][j] - mg - xh * mgx);
          }
          if (dres_in != nullptr) {
            float q[8];
            load8(dres_in + (size_t)(row0 + r) * d + vi * 8, q);
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] += q[j];
          }
          store8(dx + (size_t)(row0 + r) * d + vi * 8, o);
        }
      }
    }
  }
  if (partial != nullptr) {
    float* pw = partial + (size_t)blockIdx.x * 2 * d;
    float* pb = pw + d;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int vi = threadIdx.x + i * kNormThreads;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          pw[vi * 8 + j] = dw[i][j];
          if (WANT_DB) pb[vi * 8 + j] = db[i][j];
        }
      }
    }
  }
}

// dw[c] (+)= sum_p partial[p][0][c];  db[c] (+)= sum_p partial[p][1][c]
// Block = 32 columns x 16 part-lanes: the parts are split over the lanes and
// folded through shared memory, so the serial chain per thread is nparts / 16.
constexpr int kRedCols = 32, kRedLanes = 16;
__global__ void __launch_bounds__(kRedCols * kRedLanes)
norm_bwd_reduce_kernel(const float* __restrict__ partial, int nparts, int d,
                       float* __restrict__ dw, float* __restrict__ db, int accumulate) {
  __shared__ float s_w[kRedLanes][kRedCols + 1], s_b[kRedLanes][kRedCols + 1];
  const int col = threadIdx.x, lane = threadIdx.y;
  const int c = blockIdx.x * kRedCols + col;
  float sw = 0.f, sb = 0.f;
  if (c < d) {
    for (int p = lane; p < nparts; p += kRedLanes) {
      sw += partial[(size_t)p * 2 * d + c];
      sb += partial[(size_t)p * 2 * d + d + c];
    }
  }
  s_w[lane][col] = sw;
  s_b[lane][col] = sb;
  __syncthreads();
  if (lane == 0 && c < d) {
#pragma unroll
    for (int l = 1; l < kRedLanes; ++l) { sw += s_w[l][col]; sb += s_b[l][col]; }
    if (dw != nullptr) dw[c] = accumulate ? dw[c] + sw : sw;
    if (db != nullptr) db[c] = accumulate ? db[c] + sb : sb;
  }
}

// ---------------------------------------------------------------------------
// SwiGLU on a [rows, 2F] tensor laid out as [gate(F) | up(F)] per row.
// ---------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                  long long rows, int F) {
  const int fv = F >> 3;
  const long long total = rows * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / fv;
    const int c = (int)(i - r * fv) * 8;
    float g[8], u[8], o[8];
    load8(gu + r * 2 * F + c, g);
    load8(gu + r * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8(out + r * F + c, o);
  }
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, long long rows, int F) {
  const int fv = F >> 3;
  const long long total = rows * fv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / fv;
    const int c = (int)(i - r * fv) * 8;
    float g[8], u[8], dy[8], dg[8], du[8];
    load8(gu + r * 2 * F + c, g);
    load8(gu + r * 2 * F + F + c, u);
    load8(dout + r * F + c, dy);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * sg;
      du[j] = dy[j] * silu;
      dg[j] = dy[j] * u[j] * (sg + silu * (1.f - sg));
    }
    store8(dgu + r * 2 * F + c, dg);
    store8(dgu + r * 2 * F + F + c, du);
  }
}

// ------------------------------- GELU (tanh) -------------------------------
__device__ __forceinline__ float gelu_f(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float k = 0.7978845608028654f;
  const float t = tanhf(k * (x + 0.044715f * x * x * x));
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
}
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8], o[8];
    load8(x + i * 8, a);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gelu_f(a[j]);
    store8(y + i * 8, o);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                __nv_bfloat16* __restrict__ dx, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float a[8], g[8], o[8];
    load8(x + i * 8, a);
    load8(dy + i * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] * gelu_grad_f(a[j]);
    store8(dx + i * 8, o);
  }
}

// ---------------------------------------------------------------------------
// Rotary embedding (rotate-half convention) applied in place to the first
// `nheads` heads of a [tokens, heads_total, hd] tensor.  cs = [seq, hd/2] of
// (cos, sin) pairs; position = pos_offset + token % seq.  sign = -1 gives the
// adjoint (backward).
// ---------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float2* __restrict__ cs, long long tokens,
                            int seq, int heads_total, int nheads, int hd, float sign) {
  const int half = hd >> 1;
  const int hv = half >> 3;  // 8-element vectors per half head
  const long long total = tokens * nheads * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % hv);
    const long long th = i / hv;
    const int h = (int)(th % nheads);
    const long long t = th / nheads;
    const int pos = (int)(t % seq);
    __nv_bfloat16* p = qkv + (t * heads_total + h) * hd + v * 8;
    float a[8], b[8], oa[8], ob[8];
    load8(p, a);
    load8(p + half, b);
    const float2* c = cs + (size_t)pos * half + v * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float co = c[j].x, si = c[j].y * sign;
      oa[j] = a[j] * co - b[j] * si;
      ob[j] = b[j] * co + a[j] * si;
    }
    store8(p, oa);
    store8(p + half, ob);
  }
}

// ------------------------------- embedding ---------------------------------
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long tokens, int d, long long vocab) {
  const int dv = d >> 3;
  const long long total = tokens * dv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / dv;
    const int c = (int)(i - t * dv) * 8;
    const long long id = ids[t];
    uint4 u = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < vocab) u = *reinterpret_cast<const uint4*>(table + id * d + c);
    *reinterpret_cast<uint4*>(out + t * d + c) = u;
  }
}
// grad_table[ids[t]] += dout[t]  (fp32 accumulation buffer)
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ grad_table, long long tokens, int d, long long vocab) {
  const int dv = d >> 3;
  const long long total = tokens * dv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / dv;
    const int c = (int)(i - t * dv) * 8;
    const long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    float g[8];
    load8(dout + t * d + c, g);
    float* dst = grad_table + id * d + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dst + j, g[j]);
  }
}

// ---------------------------------------------------------------------------
// Fused softmax cross-entropy over bf16 logits [rows, ld] (first V columns
// valid).  loss[row] = lse - logit[target]; logits are overwritten by
// (softmax - onehot) * grad_scale (columns >= V get 0).  target < 0 = ignored.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
xent_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
            float* __restrict__ loss, int V, int ld, float grad_scale) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * (long long)ld;
  const int nvec = ld >> 3;
  float m = -INFINITY, s = 0.f;
  for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
    float a[8];
    load8(lr + vi * 8, a);
    float lm = m;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (vi * 8 + j < V) lm = fmaxf(lm, a[j]);
    if (lm > m) { s *= __expf(m - lm); m = lm; }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (vi * 8 + j < V) s += __expf(a[j] - m);
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  s = block_sum(s, red);
  const float lse = gm + logf(s);
  const long long tgt = targets[row];
  if (threadIdx.x == 0) loss[row] = (tgt >= 0 && tgt < V) ? lse - __bfloat162float(lr[tgt]) : 0.f;
  __syncthreads();
  const float sc = (tgt >= 0 && tgt < V) ? grad_scale : 0.f;
  for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
    float a[8], o[8];
    load8(lr + vi * 8, a);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = vi * 8 + j;
      float p = (c < V) ? __expf(a[j] - lse) : 0.f;
      if (c == tgt) p -= 1.f;
      o[j] = p * sc;
    }
    store8(lr + vi * 8, o);
  }
}

// ---------------------------------------------------------------------------
// Fused AdamW on flat buffers.  master/m/v fp32; grad fp32 (gradient
// accumulation buffer) which is cleared after use when zero_grad != 0; the
// bf16 working copy of the parameters is refreshed in the same pass.
// grad_scale_ptr (device scalar, may be null) multiplies the gradient, e.g. the
// clipping coefficient times 1/accumulation steps.
// ---------------------------------------------------------------------------
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             float* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, long long n,
                             float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ grad_scale_ptr, float grad_scale, int zero_grad) {
  const float gs = grad_scale * (grad_scale_ptr ? *grad_scale_ptr : 1.f);
  const long long nvec = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 p = reinterpret_cast<float4*>(master)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float4 g = reinterpret_cast<float4*>(grad)[i];
    float pa[4] = {p.x, p.y, p.z, p.w}, ma[4] = {mm.x, mm.y, mm.z, mm.w}, va[4] = {vv.x, vv.y, vv.z, vv.w},
          ga[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = ga[j] * gs;
      ma[j] = beta1 * ma[j] + (1.f - beta1) * gj;
      va[j] = beta2 * va[j] + (1.f - beta2) * gj * gj;
      const float mh = ma[j] / bc1, vh = va[j] / bc2;
      pa[j] = pa[j] * (1.f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(pa[0], pa[1], pa[2], pa[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(ma[0], ma[1], ma[2], ma[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(va[0], va[1], va[2], va[3]);
    if (zero_grad) reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (param_bf16 != nullptr) {
      uint2 o;
      o.x = pack_bf16x2(pa[0], pa[1]);
      o.y = pack_bf16x2(pa[2], pa[3]);
      reinterpret_cast<uint2*>(param_bf16)[i] = o;
    }
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0) {
    for (long long i = (nvec << 2) + threadIdx.x; i < n; i += blockDim.x) {
      const float gj = grad[i] * gs;
      const float mj = beta1 * m[i] + (1.f - beta1) * gj;
      const float vj = beta2 * v[i] + (1.f - beta2) * gj * gj;
      const float pj = master[i] * (1.f - lr * wd) - lr * (mj / bc1) / (sqrtf(vj / bc2) + eps);
      m[i] = mj; v[i] = vj; master[i] = pj;
      if (zero_grad) grad[i] = 0.f;
      if (param_bf16 != nullptr) param_bf16[i] = __float2bfloat16(pj);
    }
  }
}

// out[0] += sum x^2   (fp32 input)
__global__ void sumsq_f32_kernel(const float* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float a = x[i];
    s += a * a;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// y = a + b (bf16), 8 elements per thread.
__global__ void add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                __nv_bfloat16* __restrict__ y, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float x[8], z[8];
    load8(a + i * 8, x);
    load8(b + i * 8, z);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += z[j];
    store8(y + i * 8, x);
  }
}

// dst(bf16) = src(fp32) * scale
__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n,
                                     float scale) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16(src[i] * scale);
}
// dst(fp32) (+)= src(bf16) * scale
__global__ void cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n,
                                     float scale, int accumulate) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(src[i]) * scale;
    dst[i] = accumulate ? dst[i] + v : v;
  }
}

inline int grid_for(long long work, int threads, int cap_mult = 16) {
  long long b = (work + threads - 1) / threads;
  const long long cap = 148ll * cap_mult;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace

#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<__nv_bfloat16*>(p)
#define CBF(p) reinterpret_cast<const __nv_bfloat16*>(p)

// Number of CTAs the norm backward uses == rows of the partial scratch buffer.
// Rows that a CTA takes per iteration for rows of nvec 8-element vectors (see the kernels).
static inline int norm_rows_per_iter(int d) { return d <= 4096 ? 4 : 2; }

template <bool RMS>
static void launch_norm_fwd(int grid, cudaStream_t s, const void* x, const void* res, void* xsum, const void* w,
                            const void* b, void* y, void* stats, int rows, int d, float eps) {
  if (d <= 2048)
    norm_fwd_kernel<RMS, 1, 4><<<grid, kNormThreads, 0, s>>>(CBF(x), CBF(res), BF(xsum), CBF(w), CBF(b), BF(y),
                                                             (float2*)stats, rows, d, eps);
  else if (d <= 4096)
    norm_fwd_kernel<RMS, 2, 4><<<grid, kNormThreads, 0, s>>>(CBF(x), CBF(res), BF(xsum), CBF(w), CBF(b), BF(y),
                                                             (float2*)stats, rows, d, eps);
  else
    norm_fwd_kernel<RMS, 4, 2><<<grid, kNormThreads, 0, s>>>(CBF(x), CBF(res), BF(xsum), CBF(w), CBF(b), BF(y),
                                                             (float2*)stats, rows, d, eps);
}

template <bool RMS, bool WANT_DB>
static void launch_norm_bwd(int grid, cudaStream_t s, const void* dy, const void* x, const void* w, const void* stats,
                            const void* dres, void* dx, float* partial, int rows, int d) {
  if (d <= 2048)
    norm_bwd_kernel<RMS, 1, 4, WANT_DB><<<grid, kNormThreads, 0, s>>>(CBF(dy), CBF(x), CBF(w), (const float2*)stats,
                                                                      CBF(dres), BF(dx), partial, rows, d);
  else if (d <= 4096)
    norm_bwd_kernel<RMS, 2, 2, WANT_DB><<<grid, kNormThreads, 0, s>>>(CBF(dy), CBF(x), CBF(w), (const float2*)stats,
                                                                      CBF(dres), BF(dx), partial, rows, d);
  else
    norm_bwd_kernel<RMS, 4, 1, WANT_DB><<<grid, kNormThreads, 0, s>>>(CBF(dy), CBF(x), CBF(w), (const float2*)stats,
                                                                      CBF(dres), BF(dx), partial, rows, d);
}
static void launch_norm_bwd_any(int rms, bool want_db, int grid, cudaStream_t s, const void* dy, const void* x,
                                const void* w, const void* stats, const void* dres, void* dx, float* partial,
                                int rows, int d) {
  if (rms) {
    if (want_db) launch_norm_bwd<true, true>(grid, s, dy, x, w, stats, dres, dx, partial, rows, d);
    else launch_norm_bwd<true, false>(grid, s, dy, x, w, stats, dres, dx, partial, rows, d);
  } else {
    if (want_db) launch_norm_bwd<false, true>(grid, s, dy, x, w, stats, dres, dx, partial, rows, d);
    else launch_norm_bwd<false, false>(grid, s, dy, x, w, stats, dres, dx, partial, rows, d);
  }
}

// CTAs of the backward kernel = slices of its partial-sum scratch.
DD_API int dd_norm_bwd_parts(int rows) {
  const int groups = (rows + 1) / 2;
  return groups < 148 * 4 ? (groups > 0 ? groups : 1) : 148 * 4;
}

DD_API int dd_norm_fwd(int rms, const void* x, const void* res, void* xsum, const void* w, const void* b, void* y,
                       void* stats, int rows, int d, float eps, void* stream) {
  if (d % 8 != 0 || d > kNormThreads * kMaxVec * 8 || rows <= 0) return DD_ERR_BAD_ARG;
  const int groups = (rows + norm_rows_per_iter(d) - 1) / norm_rows_per_iter(d);
  const int grid = groups < 148 * 8 ? groups : 148 * 8;
  if (rms) launch_norm_fwd<true>(grid, STREAM(stream), x, res, xsum, w, b, y, stats, rows, d, eps);
  else launch_norm_fwd<false>(grid, STREAM(stream), x, res, xsum, w, b, y, stats, rows, d, eps);
  return (int)cudaGetLastError();
}

// partial: scratch of dd_norm_bwd_parts(rows) * 2 * d floats (may be null when
// neither dw nor db is wanted).
DD_API int dd_norm_bwd(int rms, const void* dy, const void* x, const void* w, const void* stats, const void* dres,
                       void* dx, float* dw, float* db, float* partial, int accumulate, int rows, int d,
                       void* stream) {
  if (d % 8 != 0 || d > kNormThreads * kMaxVec * 8 || rows <= 0) return DD_ERR_BAD_ARG;
  const int grid = dd_norm_bwd_parts(rows);
  launch_norm_bwd_any(rms, db != nullptr && partial != nullptr, grid, STREAM(stream), dy, x, w, stats, dres, dx,
                      partial, rows, d);
  if (partial != nullptr && (dw != nullptr || db != nullptr))
    norm_bwd_reduce_kernel<<<(d + kRedCols - 1) / kRedCols, dim3(kRedCols, kRedLanes), 0, STREAM(stream)>>>(partial, grid, d, dw, db, accumulate);
  return (int)cudaGetLastError();
}

DD_API int dd_swiglu_fwd(const void* gu, void* out, long long rows, int F, void* stream) {
  if (F % 8) return DD_ERR_BAD_ARG;
  swiglu_fwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, STREAM(stream)>>>(CBF(gu), BF(out), rows, F);
  return (int)cudaGetLastError();
}
DD_API int dd_swiglu_bwd(const void* dout, const void* gu, void* dgu, long long rows, int F, void* stream) {
  if (F % 8) return DD_ERR_BAD_ARG;
  swiglu_bwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, STREAM(stream)>>>(CBF(dout), CBF(gu), BF(dgu), rows, F);
  return (int)cudaGetLastError();
}
DD_API int dd_gelu_fwd(const void* x, void* y, long long n, void* stream) {
  if (n % 8) return DD_ERR_BAD_ARG;
  gelu_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, STREAM(stream)>>>(CBF(x), BF(y), n / 8);
  return (int)cudaGetLastError();
}
DD_API int dd_gelu_bwd(const void* dy, const void* x, void* dx, long long n, void* stream) {
  if (n % 8) return DD_ERR_BAD_ARG;
  gelu_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, STREAM(stream)>>>(CBF(dy), CBF(x), BF(dx), n / 8);
  return (int)cudaGetLastError();
}
DD_API int dd_rope(void* qkv, const void* cs, long long tokens, int seq, int heads_total, int nheads, int hd,
                   float sign, void* stream) {
  if (hd % 16 || nheads > heads_total) return DD_ERR_BAD_ARG;
  rope_kernel<<<grid_for(tokens * nheads * (hd / 16), 256), 256, 0, STREAM(stream)>>>(
      BF(qkv), (const float2*)cs, tokens, seq, heads_total, nheads, hd, sign);
  return (int)cudaGetLastError();
}
DD_API int dd_embedding_fwd(const void* ids, const void* table, void* out, long long tokens, int d,
                            long long vocab, void* stream) {
  if (d % 8) return DD_ERR_BAD_ARG;
  embedding_fwd_kernel<<<grid_for(tokens * (d / 8), 256), 256, 0, STREAM(stream)>>>(
      (const long long*)ids, CBF(table), BF(out), tokens, d, vocab);
  return (int)cudaGetLastError();
}
DD_API int dd_embedding_bwd(const void* ids, const void* dout, float* grad_table, long long tokens, int d,
                            long long vocab, void* stream) {
  if (d % 8) return DD_ERR_BAD_ARG;
  embedding_bwd_kernel<<<grid_for(tokens * (d / 8), 256), 256, 0, STREAM(stream)>>>(
      (const long long*)ids, CBF(dout), grad_table, tokens, d, vocab);
  return (int)cudaGetLastError();
}
DD_API int dd_xent(void* logits, const void* targets, float* loss, long long rows, int V, int ld,
                   float grad_scale, void* stream) {
  if (ld % 8 || V > ld || rows <= 0) return DD_ERR_BAD_ARG;
  xent_kernel<<<(unsigned)rows, 1024, 0, STREAM(stream)>>>(BF(logits), (const long long*)targets, loss, V, ld,
                                                          grad_scale);
  return (int)cudaGetLastError();
}
DD_API int dd_adamw(float* master, float* m, float* v, float* grad, void* param_bf16, long long n, float lr,
                    float beta1, float beta2, float eps, float wd, int step, const float* grad_scale_ptr,
                    float grad_scale, int zero_grad, void* stream) {
  if (n <= 0) return DD_OK;
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(grad)) & 15)
    return DD_ERR_ALIGN;
  if (reinterpret_cast<uintptr_t>(param_bf16) & 7) return DD_ERR_ALIGN;
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  adamw_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, STREAM(stream)>>>(master, m, v, grad, BF(param_bf16), n, lr,
                                                                      beta1, beta2, eps, wd, bc1, bc2,
                                                                      grad_scale_ptr, grad_scale, zero_grad);
  return (int)cudaGetLastError();
}
DD_API int dd_sumsq_f32(const float* x, long long n, float* out, void* stream) {
  if (n <= 0) return DD_OK;
  sumsq_f32_kernel<<<grid_for(n, 256, 8), 256, 0, STREAM(stream)>>>(x, n, out);
  return (int)cudaGetLastError();
}
DD_API int dd_add_bf16(const void* a, const void* b, void* y, long long n, void* stream) {
  if (n % 8) return DD_ERR_BAD_ARG;
  add_bf16_kernel<<<grid_for(n / 8, 256), 256, 0, STREAM(stream)>>>(CBF(a), CBF(b), BF(y), n / 8);
  return (int)cudaGetLastError();
}
DD_API int dd_cast_f32_bf16(const float* src, void* dst, long long n, float scale, void* stream) {
  if (n <= 0) return DD_OK;
  cast_f32_bf16_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(src, BF(dst), n, scale);
  return (int)cudaGetLastError();
}
DD_API int dd_cast_bf16_f32(const void* src, float* dst, long long n, float scale, int accumulate, void* stream) {
  if (n <= 0) return DD_OK;
  cast_bf16_f32_kernel<<<grid_for(n, 256), 256, 0, STREAM(stream)>>>(CBF(src), dst, n, scale, accumulate);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Norm backward without any allocation (declared in no_alloc.h).
//
// Same kernels as dd_norm_bwd, but the per-CTA partial sums of dw / db go to a
// fixed array that is part of the loaded library instead of a buffer the caller
// allocates.  For callers that are not able to allocate device memory at the
// time of the call: a plug-in or custom-call hook inside a host program that
// reserved the whole device up front (a later cudaMalloc there simply fails),
// or a latency-critical section in which the implicit device synchronisation of
// cudaMalloc / cudaFree is not acceptable.
// ---------------------------------------------------------------------------
namespace {
constexpr int kNoAllocMaxD = kNormThreads * kMaxVec * 8;   // 8192 columns
constexpr int kNoAllocParts = 148;                          // one partial row pair per SM
// 148 * 2 * 8192 floats = 9.25 MiB, resident on every GPU that loads the library.
static __device__ __align__(256) float g_norm_bwd_scratch[(size_t)kNoAllocParts * 2 * kNoAllocMaxD];
float* g_norm_bwd_scratch_addr[64] = {nullptr};
}  // namespace

DD_API int dd_norm_bwd_noalloc_max_d() { return kNoAllocMaxD; }
DD_API long long dd_norm_bwd_noalloc_scratch_bytes() { return (long long)sizeof(float) * kNoAllocParts * 2 * kNoAllocMaxD; }

DD_API int dd_norm_bwd_noalloc(int rms, const void* dy, const void* x, const void* w, const void* stats, void* dx,
                               float* dw, float* db, int accumulate, int rows, int d, void* stream) {
  if (rows <= 0 || d <= 0 || d % 8 != 0) {
    fprintf(stderr, "dd_norm_bwd_noalloc: rows must be positive and d a positive multiple of 8 (rows=%d, d=%d)\n",
            rows, d);
    return DD_ERR_BAD_ARG;
  }
  if (d > kNoAllocMaxD) {
    fprintf(stderr, "dd_norm_bwd_noalloc: d=%d exceeds the built-in scratch (at most %d columns)\n", d, kNoAllocMaxD);
    return DD_ERR_TOO_LARGE;
  }
  // Argument checks before anything is launched, as in the other entry points:
  // a null or misaligned pointer would otherwise fault inside the kernel.
  if (dy == nullptr || x == nullptr || stats == nullptr || dx == nullptr) {
    fprintf(stderr, "dd_norm_bwd_noalloc: dy, x, stats and dx must not be null\n");
    return DD_ERR_BAD_ARG;
  }
  if (((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx) |
        reinterpret_cast<uintptr_t>(w)) & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(stats) & 7) != 0 ||
      ((reinterpret_cast<uintptr_t>(dw) | reinterpret_cast<uintptr_t>(db)) & 3) != 0) {
    fprintf(stderr, "dd_norm_bwd_noalloc: dy, x, w and dx need 16-byte alignment, stats 8, dw and db 4\n");
    return DD_ERR_ALIGN;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return DD_ERR_BAD_ARG;
  // One-time set-up per device, with that device current: in host code the
  // array's name is only a handle, the device address has to be looked up.
  // The cache is written without a lock: two threads that race here both look
  // up and store the same address, which is harmless.
  if (g_norm_bwd_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_norm_bwd_scratch);
    if (e != cudaSuccess) return (int)e;
    g_norm_bwd_scratch_addr[dev] = p;
  }
  // Without dw and db the partial sums are not wanted: the kernel then skips them.
  float* partial = (dw != nullptr || db != nullptr) ? g_norm_bwd_scratch_addr[dev] : nullptr;
  const int grid = rows < kNoAllocParts ? rows : kNoAllocParts;
  // Every CTA overwrites its whole [2][d] slice of the scratch, so nothing left
  // by an earlier call is ever read: no clearing is needed.
  launch_norm_bwd_any(rms, db != nullptr, grid, STREAM(stream), dy, x, w, stats, nullptr, dx, partial, rows, d);
  if (dw != nullptr || db != nullptr)
    norm_bwd_reduce_kernel<<<(d + kRedCols - 1) / kRedCols, dim3(kRedCols, kRedLanes), 0, STREAM(stream)>>>(partial, grid, d, dw, db, accumulate);
  return (int)cudaGetLastError();
}
