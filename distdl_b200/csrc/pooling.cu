// Local arithmetic of the distributed pooling layers: average and max pooling of
// [planes, n0, n1, n2] tensors (planes = batch x channels; 1-D and 2-D pooling use leading
// extents of 1), fp32 or bf16, no padding (the layer pads at the global boundary and
// exchanges halos first, nn/pooling.py).  The input may be a strided view (the cropped
// interior of the halo-exchanged tensor), so the crop costs no copy; outputs are contiguous.
// The reference calls torch.nn.functional.{avg,max}_pool{1,2,3}d on a contiguous crop here
// (src/distdl/nn/pooling.py:150-170).
//
//   forward : one thread per output element walks its window (dilated for max pooling);
//             max pooling also records the input position of the maximum (the first of equal
//             values wins, a NaN wins over everything, as in PyTorch).
//   backward: one thread per INPUT element gathers from the outputs whose windows cover it
//             (no atomics, deterministic); dx is contiguous with the shape of the view.
#include "common.cuh"

using namespace dd;

namespace {

struct PoolGeom {
  long long planes;
  int in[3], out[3], k[3], s[3], d[3];
  long long xs_plane, xs[3];      // element strides of the input view
};

template <typename T> __device__ __forceinline__ float pf(T v);
template <> __device__ __forceinline__ float pf<float>(float v) { return v; }
template <> __device__ __forceinline__ float pf<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T pt(float v);
template <> __device__ __forceinline__ float pt<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 pt<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

template <typename T, bool MAX>
__global__ void __launch_bounds__(256)
pool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int* __restrict__ arg, const PoolGeom g, float inv_vol) {
  const long long per_plane = (long long)g.out[0] * g.out[1] * g.out[2];
  const long long total = g.planes * per_plane;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long pl = e / per_plane;
    long long r = e - pl * per_plane;
    const int o0 = (int)(r / ((long long)g.out[1] * g.out[2]));
    r -= (long long)o0 * g.out[1] * g.out[2];
    const int o1 = (int)(r / g.out[2]), o2 = (int)(r - (long long)o1 * g.out[2]);
    const T* xp = x + pl * g.xs_plane;
    float acc = MAX ? -INFINITY : 0.f;
    int best = -1;
    for (int a = 0; a < g.k[0]; ++a) {
      const int i0 = o0 * g.s[0] + a * g.d[0];
      for (int b = 0; b < g.k[1]; ++b) {
        const int i1 = o1 * g.s[1] + b * g.d[1];
        for (int c = 0; c < g.k[2]; ++c) {
          const int i2 = o2 * g.s[2] + c * g.d[2];
          const float v = pf<T>(xp[i0 * g.xs[0] + i1 * g.xs[1] + i2 * g.xs[2]]);
          if (MAX) {
            const int idx = (i0 * g.in[1] + i1) * g.in[2] + i2;
            if (best < 0) best = idx;
            if (v > acc || v != v) { acc = v; best = idx; }
          } else {
            acc += v;
          }
        }
      }
    }
    y[e] = pt<T>(MAX ? acc : acc * inv_vol);
    if (MAX) arg[e] = best;
  }
}

// outputs o with o * s + a * d == i for some 0 <= a < k, o in [0, n_out): the range of candidates
__device__ __forceinline__ void cover(int i, int k, int s, int d, int n_out, int& lo, int& hi) {
  const int first = i - (k - 1) * d;                         // smallest window start that still reaches i
  lo = first <= 0 ? 0 : (first + s - 1) / s;
  hi = i / s;
  if (hi > n_out - 1) hi = n_out - 1;
}

template <typename T, bool MAX>
__global__ void __launch_bounds__(256)
pool_bwd_kernel(const T* __restrict__ dy, const int* __restrict__ arg, T* __restrict__ dx, const PoolGeom g,
                float inv_vol) {
  const long long per_plane = (long long)g.in[0] * g.in[1] * g.in[2];
  const long long out_plane = (long long)g.out[0] * g.out[1] * g.out[2];
  const long long total = g.planes * per_plane;
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const long long pl = e / per_plane;
    long long r = e - pl * per_plane;
    const int here = (int)r;
    const int i0 = (int)(r / ((long long)g.in[1] * g.in[2]));
    r -= (long long)i0 * g.in[1] * g.in[2];
    const int i1 = (int)(r / g.in[2]), i2 = (int)(r - (long long)i1 * g.in[2]);
    int lo0, hi0, lo1, hi1, lo2, hi2;
    cover(i0, g.k[0], g.s[0], g.d[0], g.out[0], lo0, hi0);
    cover(i1, g.k[1], g.s[1], g.d[1], g.out[1], lo1, hi1);
    cover(i2, g.k[2], g.s[2], g.d[2], g.out[2], lo2, hi2);
    const T* dyp = dy + pl * out_plane;
    const int* ap = MAX ? arg + pl * out_plane : nullptr;
    float acc = 0.f;
    for (int o0 = lo0; o0 <= hi0; ++o0) {
      if ((i0 - o0 * g.s[0]) % g.d[0]) continue;
      for (int o1 = lo1; o1 <= hi1; ++o1) {
        if ((i1 - o1 * g.s[1]) % g.d[1]) continue;
        for (int o2 = lo2; o2 <= hi2; ++o2) {
          if ((i2 - o2 * g.s[2]) % g.d[2]) continue;
          const long long o = ((long long)o0 * g.out[1] + o1) * g.out[2] + o2;
          if (MAX) {
            if (ap[o] == here) acc += pf<T>(dyp[o]);
          } else {
            acc += pf<T>(dyp[o]);
          }
        }
      }
    }
    dx[e] = pt<T>(MAX ? acc : acc * inv_vol);
  }
}

int fill(PoolGeom& g, long long planes, const int* in, const int* out, const int* k, const int* s, const int* d,
         long long xs_plane, const long long* xs) {
  if (planes <= 0) return DD_ERR_BAD_ARG;
  g.planes = planes;
  g.xs_plane = xs_plane;
  for (int i = 0; i < 3; ++i) {
    if (in[i] <= 0 || out[i] <= 0 || k[i] <= 0 || s[i] <= 0 || d[i] <= 0) return DD_ERR_BAD_ARG;
    if ((long long)(out[i] - 1) * s[i] + (long long)(k[i] - 1) * d[i] >= in[i]) return DD_ERR_BAD_ARG;   // window leaves the input
    g.in[i] = in[i]; g.out[i] = out[i]; g.k[i] = k[i]; g.s[i] = s[i]; g.d[i] = d[i];
    g.xs[i] = xs ? xs[i] : 0;
  }
  if ((long long)in[0] * in[1] * in[2] > 0x7fffffffLL) return DD_ERR_TOO_LARGE;   // window positions are int32
  return 0;
}

unsigned grid_for(long long total) {
  long long b = (total + 255) / 256;
  if (b > 148 * 16) b = 148 * 16;
  return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace

// dtype: 0 = bf16, 1 = fp32; is_max: 0 = average (divides by the window volume), 1 = max.
// x: strided view [planes, in0, in1, in2] (xs_plane / xs: element strides); y: contiguous
// [planes, out0, out1, out2]; arg (max only): int32, same shape as y.
DD_API int dd_pool_fwd(const void* x, void* y, int* arg, long long planes, const int* in, const int* out, const int* k,
                       const int* s, const int* d, long long xs_plane, const long long* xs, int is_max, int dtype,
                       void* stream) {
  PoolGeom g;
  int r = fill(g, planes, in, out, k, s, d, xs_plane, xs);
  if (r) return r;
  if (x == nullptr || y == nullptr || (is_max && arg == nullptr)) return DD_ERR_BAD_ARG;
  const float inv = 1.f / ((float)k[0] * k[1] * k[2]);
  const long long total = planes * out[0] * out[1] * out[2];
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = grid_for(total);
#define DD_POOL_FWD(T, M) pool_fwd_kernel<T, M><<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(x), reinterpret_cast<T*>(y), arg, g, inv)
  if (dtype == 0) { if (is_max) DD_POOL_FWD(__nv_bfloat16, true); else DD_POOL_FWD(__nv_bfloat16, false); }
  else            { if (is_max) DD_POOL_FWD(float, true); else DD_POOL_FWD(float, false); }
#undef DD_POOL_FWD
  return (int)cudaGetLastError();
}

// dy / arg: contiguous [planes, out...]; dx: contiguous [planes, in...] (the shape of the view x was).
DD_API int dd_pool_bwd(const void* dy, const int* arg, void* dx, long long planes, const int* in, const int* out,
                       const int* k, const int* s, const int* d, int is_max, int dtype, void* stream) {
  PoolGeom g;
  int r = fill(g, planes, in, out, k, s, d, 0, nullptr);
  if (r) return r;
  if (dy == nullptr || dx == nullptr || (is_max && arg == nullptr)) return DD_ERR_BAD_ARG;
  const float inv = 1.f / ((float)k[0] * k[1] * k[2]);
  const long long total = planes * in[0] * in[1] * in[2];
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = grid_for(total);
#define DD_POOL_BWD(T, M) pool_bwd_kernel<T, M><<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(dy), arg, reinterpret_cast<T*>(dx), g, inv)
  if (dtype == 0) { if (is_max) DD_POOL_BWD(__nv_bfloat16, true); else DD_POOL_BWD(__nv_bfloat16, false); }
  else            { if (is_max) DD_POOL_BWD(float, true); else DD_POOL_BWD(float, false); }
#undef DD_POOL_BWD
  return (int)cudaGetLastError();
}
