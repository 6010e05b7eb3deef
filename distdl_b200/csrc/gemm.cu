// C entry point of the tcgen05 GEMM.
#include <cstdlib>

#include "gemm2_tcgen05.cuh"
#include <cstring>

#include "gemm_tcgen05.cuh"
#include "runtime.cuh"

using namespace dd;
using namespace dd::gemm;

namespace {
template <bool A_MN, bool B_MN>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int grid, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_bf16_kernel<A_MN, B_MN>;
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  kern<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}
template <bool A_MN, bool B_MN>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const Params& p, int grid,
                cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = dd::gemm2::gemm2_bf16_kernel<A_MN, B_MN>;
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dd::gemm2::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  kern<<<grid, dd::gemm2::NUM_THREADS, dd::gemm2::SMEM_BYTES, stream>>>(ta, tb, td, p);
  return (int)cudaGetLastError();
}
}  // namespace

// D[b,m,n] (+)= sum_k A[b,m,k] B[b,n,k] (+ bias[n]);  bf16 operands, fp32 accumulation.
//   a_mn / b_mn : 0 = K-major (lda = elements between rows m / n),
//                 1 = MN-major (lda = elements between rows k)
//   stride*     : elements between batches (ignored when batch == 1)
//   flags       : dd::gemm::Flags
//   max_ctas    : 0 = one CTA per SM; otherwise an upper bound (used to leave
//                 SMs to a concurrent communication kernel)
DD_API int dd_gemm_bf16(const void* A, int a_mn, long long lda, long long strideA, const void* B, int b_mn,
                        long long ldb, long long strideB, void* D, long long ldd, long long strideD,
                        const void* bias, int M, int N, int K, int batch, int flags, int max_ctas,
                        void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return DD_ERR_BAD_ARG;
  if ((lda % 8) || (ldb % 8)) return DD_ERR_ALIGN;
  if (batch > 1 && ((strideA % 8) || (strideB % 8))) return DD_ERR_ALIGN;
  if (batch == 1) {
    strideA = (a_mn ? (long long)K : (long long)M) * lda;
    strideB = (b_mn ? (long long)K : (long long)N) * ldb;
    strideD = (long long)M * ldd;
  }
  // CTA pairs (cta_group::2) unless disabled or the problem is a single tile row
  static const bool pair_ok = []() { const char* e = getenv("DISTDL_GEMM_PAIR"); return !(e && e[0] == '0'); }();
  if (pair_ok && M > BM) {
    CUtensorMap pa, pb;
    int rr;
    namespace g2 = dd::gemm2;
    if (a_mn) rr = get_tensor_map_bf16_3d(&pa, A, M, K, batch, lda * 2, strideA * 2, 64, g2::BK);
    else      rr = get_tensor_map_bf16_3d(&pa, A, K, M, batch, lda * 2, strideA * 2, g2::BK, g2::BM);
    if (rr) return rr;
    if (b_mn) rr = get_tensor_map_bf16_3d(&pb, B, N, K, batch, ldb * 2, strideB * 2, 64, g2::BK);
    else      rr = get_tensor_map_bf16_3d(&pb, B, K, N, batch, ldb * 2, strideB * 2, g2::BK, g2::BNH);
    if (rr) return rr;
    int err2 = 0;
    Params q;
    q.M = M; q.N = N; q.K = K; q.batch = batch;
    q.D = D; q.ldd = ldd; q.strideD = strideD; q.bias = bias; q.flags = flags; q.group_m = 4;
    q.status = device_status(&err2);
    if (err2) return err2;
    const int ptiles = ((M + 2 * g2::BM - 1) / (2 * g2::BM)) * ((N + g2::BN - 1) / g2::BN) * batch;
    int ctas = current_sm_count() & ~1;
    if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas & ~1;
    if (ctas < 2) ctas = 2;
    const int pgrid = 2 * ptiles < ctas ? 2 * ptiles : ctas;
    cudaStream_t ps = reinterpret_cast<cudaStream_t>(stream);
    // TMA epilogue where the output qualifies: bf16 store, fp32 store or fp32 add
    static const bool tma_epi = []() { const char* e = getenv("DISTDL_GEMM_TMA_EPI"); return !(e && e[0] == '0'); }();
    CUtensorMap pd;
    memset(&pd, 0, sizeof(pd));
    const bool f32 = (flags & F_OUT_F32) != 0;
    const long long es = f32 ? 4 : 2;
    if (tma_epi && (f32 || !(flags & F_ACCUMULATE)) && (reinterpret_cast<uintptr_t>(D) & 15) == 0 &&
        (ldd * es) % 16 == 0 && (strideD * es) % 16 == 0) {
      rr = f32 ? get_tensor_map_f32_3d(&pd, D, N, M, batch, ldd * 4, strideD * 4, 32, 32)
               : get_tensor_map_bf16_3d(&pd, D, N, M, batch, ldd * 2, strideD * 2, 64, 32);
      if (rr) return rr;
      q.flags |= F_TMA_EPI;
    }
    if (a_mn && b_mn) return launch_pair<true, true>(pa, pb, pd, q, pgrid, ps);
    if (a_mn) return launch_pair<true, false>(pa, pb, pd, q, pgrid, ps);
    if (b_mn) return launch_pair<false, true>(pa, pb, pd, q, pgrid, ps);
    return launch_pair<false, false>(pa, pb, pd, q, pgrid, ps);
  }
  CUtensorMap ta, tb;
  int r;
  if (a_mn) r = get_tensor_map_bf16_3d(&ta, A, M, K, batch, lda * 2, strideA * 2, 64, BK);
  else      r = get_tensor_map_bf16_3d(&ta, A, K, M, batch, lda * 2, strideA * 2, BK, BM);
  if (r) return r;
  if (b_mn) r = get_tensor_map_bf16_3d(&tb, B, N, K, batch, ldb * 2, strideB * 2, 64, BK);
  else      r = get_tensor_map_bf16_3d(&tb, B, K, N, batch, ldb * 2, strideB * 2, BK, BN);
  if (r) return r;

  int err = 0;
  Params p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.D = D; p.ldd = ldd; p.strideD = strideD;
  p.bias = bias; p.flags = flags;
  p.group_m = 8;
  p.status = device_status(&err);
  if (err) return err;

  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * batch;
  int ctas = current_sm_count();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  const int grid = tiles < ctas ? tiles : ctas;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a_mn && b_mn) return launch<true, true>(ta, tb, p, grid, s);
  if (a_mn) return launch<true, false>(ta, tb, p, grid, s);
  if (b_mn) return launch<false, true>(ta, tb, p, grid, s);
  return launch<false, false>(ta, tb, p, grid, s);
}
