// Nearest-left ("constant") and multilinear interpolation of sub-tensors in
// GLOBAL coordinates, forward and adjoint, 1-3 spatial dimensions, fp32 / fp64:
// sm_100a kernels plus an OpenMP CPU implementation in the same library (the
// CPU path is the oracle of the GPU tests and serves CPU tensors).
//
// A worker holds the slab [x_off, x_off + in_local) of a global input of extent
// in_global and produces the slab [y_off, y_off + out_local) of the global
// output; index arithmetic uses the global extents, so the shards of a
// partitioned tensor reproduce the serial result exactly.  Conventions are those
// of torch.nn.functional.interpolate: with align_corners the source coordinate
// of output i is i * (in - 1) / (out - 1); otherwise max(0, (i + 0.5) * s - 0.5)
// with s = 1 / scale_factor (or in / out); nearest takes floor(i * s).
// Counterpart of the reference's CPU-only C++ extension
// (src/distdl/functional/interpolate/src/*.cpp); the adjoint on the GPU
// scatters with atomic adds.
#include <cmath>
#include <cstdint>

#include "common.cuh"

namespace {

struct InterpGeom {
  int in_local[3], out_local[3], x_off[3], y_off[3], in_global[3], out_global[3];
  double scale[3];      // source step per output index (already inverted)
  int align_corners;
  int linear;
};

template <typename T>
__host__ __device__ inline void source_index(const InterpGeom& g, int d, int o_local, int& i0, int& i1, T& lam) {
  const int og = o_local + g.y_off[d];
  const int n_in = g.in_global[d], n_out = g.out_global[d];
  if (!g.linear) {
    int idx = (int)floor((double)og * g.scale[d]);
    if (idx > n_in - 1) idx = n_in - 1;
    i0 = i1 = idx - g.x_off[d];
    lam = (T)0;
    return;
  }
  double src;
  if (g.align_corners) src = (n_out > 1) ? (double)og * (double)(n_in - 1) / (double)(n_out - 1) : 0.0;
  else {
    src = ((double)og + 0.5) * g.scale[d] - 0.5;
    if (src < 0.0) src = 0.0;
  }
  int lo = (int)floor(src);
  if (lo > n_in - 1) lo = n_in - 1;
  const int hi = lo + 1 < n_in ? lo + 1 : lo;
  double l = src - (double)lo;
  if (l < 0.0) l = 0.0;
  if (l > 1.0) l = 1.0;
  if (hi == lo) l = 0.0;
  i0 = lo - g.x_off[d];
  i1 = hi - g.x_off[d];
  lam = (T)l;
}

// One output element: gathers (forward) or scatters (adjoint) its <= 8 corners.
template <typename T, bool ADJOINT, bool ATOMIC>
__host__ __device__ inline void process_output(const InterpGeom& g, T* x, T* y, long long bc, int o0, int o1, int o2) {
  int a0[3], a1[3];
  T lam[3];
  source_index<T>(g, 0, o0, a0[0], a1[0], lam[0]);
  source_index<T>(g, 1, o1, a0[1], a1[1], lam[1]);
  source_index<T>(g, 2, o2, a0[2], a1[2], lam[2]);
  const long long in_plane = (long long)g.in_local[0] * g.in_local[1] * g.in_local[2];
  const long long out_plane = (long long)g.out_local[0] * g.out_local[1] * g.out_local[2];
  T* xb = x + bc * in_plane;
  T* yo = y + bc * out_plane + ((long long)o0 * g.out_local[1] + o1) * g.out_local[2] + o2;
  T acc = (T)0;
  const T gy = ADJOINT ? *yo : (T)0;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int s0 = c & 1, s1 = (c >> 1) & 1, s2 = (c >> 2) & 1;
    const T w = (s0 ? lam[0] : (T)1 - lam[0]) * (s1 ? lam[1] : (T)1 - lam[1]) * (s2 ? lam[2] : (T)1 - lam[2]);
    if (w == (T)0) continue;
    const int i0 = s0 ? a1[0] : a0[0], i1 = s1 ? a1[1] : a0[1], i2 = s2 ? a1[2] : a0[2];
    if (i0 < 0 || i0 >= g.in_local[0] || i1 < 0 || i1 >= g.in_local[1] || i2 < 0 || i2 >= g.in_local[2]) continue;
    T* px = xb + ((long long)i0 * g.in_local[1] + i1) * g.in_local[2] + i2;
    if (ADJOINT) {
#ifdef __CUDA_ARCH__
      if (ATOMIC) atomicAdd(px, w * gy); else *px += w * gy;
#else
      *px += w * gy;
#endif
    } else {
      acc += w * *px;
    }
  }
  if (!ADJOINT) *yo = acc;
}

template <typename T, bool ADJOINT>
__global__ void interp_kernel(const InterpGeom g, T* x, T* y, long long BC) {
  const long long out_plane = (long long)g.out_local[0] * g.out_local[1] * g.out_local[2];
  const long long total = BC * out_plane;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long bc = i / out_plane;
    long long r = i - bc * out_plane;
    const int o2 = (int)(r % g.out_local[2]); r /= g.out_local[2];
    const int o1 = (int)(r % g.out_local[1]);
    const int o0 = (int)(r / g.out_local[1]);
    process_output<T, ADJOINT, true>(g, x, y, bc, o0, o1, o2);
  }
}

template <typename T, bool ADJOINT>
void interp_cpu(const InterpGeom& g, T* x, T* y, long long BC) {
  // parallel over batch*channel planes: the adjoint's scatter never crosses planes
#pragma omp parallel for schedule(static)
  for (long long bc = 0; bc < BC; ++bc)
    for (int o0 = 0; o0 < g.out_local[0]; ++o0)
      for (int o1 = 0; o1 < g.out_local[1]; ++o1)
        for (int o2 = 0; o2 < g.out_local[2]; ++o2) process_output<T, ADJOINT, false>(g, x, y, bc, o0, o1, o2);
}

template <typename T>
int run(int cuda, int adjoint, const InterpGeom& g, void* x, void* y, long long BC, void* stream) {
  T* xp = reinterpret_cast<T*>(x);
  T* yp = reinterpret_cast<T*>(y);
  if (!cuda) {
    if (adjoint) interp_cpu<T, true>(g, xp, yp, BC); else interp_cpu<T, false>(g, xp, yp, BC);
    return 0;
  }
  const long long total = BC * g.out_local[0] * g.out_local[1] * g.out_local[2];
  if (total <= 0) return 0;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (adjoint) interp_kernel<T, true><<<(int)blocks, 256, 0, s>>>(g, xp, yp, BC);
  else interp_kernel<T, false><<<(int)blocks, 256, 0, s>>>(g, xp, yp, BC);
  return (int)cudaGetLastError();
}

}  // namespace

// nd in 1..3; all int arrays have nd entries; scale[d] = source step per output
// index (1 / scale_factor, or in_global / out_global).  Forward: y = I(x).
// Adjoint: x += I^T(y) (the caller zeroes x).  dtype: 0 fp32, 1 fp64.
DD_API int dd_interpolate(int cuda, int linear, int adjoint, int dtype, int nd, void* x, void* y, long long BC,
                          const int* in_local, const int* out_local, const int* x_off, const int* y_off,
                          const int* in_global, const int* out_global, const double* scale, int align_corners,
                          void* stream) {
  if (nd < 1 || nd > 3 || BC < 0) return DD_ERR_BAD_ARG;
  InterpGeom g;
  for (int d = 0; d < 3; ++d) {
    const int s = d - (3 - nd);     // leading dims are padded with extent 1
    if (s < 0) {
      g.in_local[d] = g.out_local[d] = g.in_global[d] = g.out_global[d] = 1;
      g.x_off[d] = g.y_off[d] = 0;
      g.scale[d] = 1.0;
    } else {
      g.in_local[d] = in_local[s]; g.out_local[d] = out_local[s];
      g.x_off[d] = x_off[s]; g.y_off[d] = y_off[s];
      g.in_global[d] = in_global[s]; g.out_global[d] = out_global[s];
      g.scale[d] = scale[s];
    }
  }
  g.align_corners = align_corners;
  g.linear = linear;
  return dtype == 0 ? run<float>(cuda, adjoint, g, x, y, BC, stream) : run<double>(cuda, adjoint, g, x, y, BC, stream);
}
