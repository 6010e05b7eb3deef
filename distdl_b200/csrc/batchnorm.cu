// Local arithmetic of the distributed batch norm on [batch, feature, rest...] tensors
// (contiguous, fp32 or bf16): per-feature reductions and the per-feature affine map.
// The layer (nn/batchnorm.py) exchanges the per-feature sums between workers with the
// SumReduce / Broadcast primitives; these kernels stand where the reference calls
// tensor.sum / elementwise PyTorch ops around those primitives
// (src/distdl/nn/batchnorm.py:306-360).
//
//   bn_reduce:  out[f]   (+)= sum over (b, r) of  u           u = x                (mode 0)
//               out2[f]  (+)= sum over (b, r) of  u * u       u = x - shift[f]     (mode 1)
//                                                 dy, dy * (x - shift[f])          (mode 2: out, out2)
//   bn_affine:  y = a[f] * (x - m[f]) + c[f]  (+ e[f] * z)   with optional second input z
// Reductions are two-level: a CTA reduces a slab of one feature in fp32 and adds its
// partial sums with one atomicAdd per output; `out` / `out2` must be zero on entry.
#include "common.cuh"

using namespace dd;

namespace {

constexpr int kBnThreads = 256;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

__device__ __forceinline__ float block_sum_bn(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (kBnThreads >> 5)) ? red[lane] : 0.f;
  return warp_sum(t);
}

// grid = (F, splits): CTA (f, s) reduces the elements e = s * blockDim + tid, stepping by
// splits * blockDim, of feature f's B * R elements (element e = (b, r) with b = e / R).
template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_reduce_kernel(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ shift, int B, int F,
                 long long R, int mode, float* __restrict__ out, float* __restrict__ out2) {
  __shared__ float red[32];
  const int f = blockIdx.x;
  const long long n = (long long)B * R;
  const float sh = (mode != 0 && shift != nullptr) ? shift[f] : 0.f;
  float a1 = 0.f, a2 = 0.f;
  for (long long e = (long long)blockIdx.y * blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.y * blockDim.x) {
    const long long b = e / R, r = e - b * R;
    const long long idx = (b * F + f) * R + r;
    const float u = to_f<T>(x[idx]) - sh;
    if (mode == 0) {
      a1 += u;
    } else if (mode == 1) {
      a1 += u;
      a2 += u * u;
    } else {
      const float g = to_f<T>(dy[idx]);
      a1 += g;
      a2 += g * u;
    }
  }
  a1 = block_sum_bn(a1, red);
  if (mode != 0) a2 = block_sum_bn(a2, red);
  if (threadIdx.x == 0) {
    atomicAdd(out + f, a1);
    if (mode != 0 && out2 != nullptr) atomicAdd(out2 + f, a2);
  }
}

template <typename T>
__global__ void __launch_bounds__(kBnThreads)
bn_affine_kernel(const T* __restrict__ x, const T* __restrict__ z, const float* __restrict__ a,
                 const float* __restrict__ m, const float* __restrict__ c, const float* __restrict__ e, int F,
                 long long R, long long total, T* __restrict__ y) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int f = (int)((i / R) % F);
    float v = a[f] * (to_f<T>(x[i]) - (m ? m[f] : 0.f)) + (c ? c[f] : 0.f);
    if (z != nullptr) v += e[f] * to_f<T>(z[i]);
    y[i] = from_f<T>(v);
  }
}

}  // namespace

// dtype: 0 = bf16, 1 = fp32.  x (and dy in mode 2): [B, F, R] contiguous; shift: [F] fp32 or null;
// out / out2: [F] fp32, zero on entry.
DD_API int dd_bn_reduce(const void* x, const void* dy, const float* shift, int B, int F, long long R, int mode,
                        int dtype, float* out, float* out2, void* stream) {
  if (B <= 0 || F <= 0 || R <= 0 || mode < 0 || mode > 2 || out == nullptr) return DD_ERR_BAD_ARG;
  if (mode == 2 && dy == nullptr) return DD_ERR_BAD_ARG;
  const long long n = (long long)B * R;
  long long splits = (n + kBnThreads * 8 - 1) / (kBnThreads * 8);
  const long long want = (148 * 8 + F - 1) / F;          // enough CTAs to fill the GPU
  if (splits > want) splits = want;
  if (splits < 1) splits = 1;
  if (splits > 65535) splits = 65535;
  dim3 grid((unsigned)F, (unsigned)splits);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 0)
    bn_reduce_kernel<__nv_bfloat16><<<grid, kBnThreads, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                                reinterpret_cast<const __nv_bfloat16*>(dy), shift, B, F,
                                                                R, mode, out, out2);
  else
    bn_reduce_kernel<float><<<grid, kBnThreads, 0, s>>>(reinterpret_cast<const float*>(x),
                                                        reinterpret_cast<const float*>(dy), shift, B, F, R, mode, out,
                                                        out2);
  return (int)cudaGetLastError();
}

// y = a[f] * (x - m[f]) + c[f] (+ e[f] * z); m, c may be null (0); z / e null together.
DD_API int dd_bn_affine(const void* x, const void* z, const float* a, const float* m, const float* c, const float* e,
                        int B, int F, long long R, int dtype, void* y, void* stream) {
  if (B <= 0 || F <= 0 || R <= 0 || a == nullptr || (z != nullptr) != (e != nullptr)) return DD_ERR_BAD_ARG;
  const long long total = (long long)B * F * R;
  long long blocks = (total + kBnThreads - 1) / kBnThreads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 0)
    bn_affine_kernel<__nv_bfloat16><<<(unsigned)blocks, kBnThreads, 0, s>>>(
        reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(z), a, m, c, e, F, R, total,
        reinterpret_cast<__nv_bfloat16*>(y));
  else
    bn_affine_kernel<float><<<(unsigned)blocks, kBnThreads, 0, s>>>(reinterpret_cast<const float*>(x),
                                                                    reinterpret_cast<const float*>(z), a, m, c, e, F, R,
                                                                    total, reinterpret_cast<float*>(y));
  return (int)cudaGetLastError();
}
