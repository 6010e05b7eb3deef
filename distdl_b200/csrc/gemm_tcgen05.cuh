// Persistent, warp-specialised bf16 GEMM for sm_100a on tcgen05 / TMEM / TMA.
//
//   D[b][m][n] (+)= sum_k A[b][m][k] * B[b][n][k]  (+ bias[n])
//
// Each operand is either K-major (k contiguous in memory) or MN-major (m resp.
// n contiguous); the four combinations cover forward (x W^T), data-gradient
// (dy W) and weight-gradient (dy^T x) GEMMs of a linear layer without any
// transposition pass.  One CTA per SM loops over 128x256 output tiles:
//
//   warp 0      TMA producer: 128B-swizzled tiles global -> shared, 4-stage ring
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (128x256x16),
//               accumulators live in TMEM, two accumulator buffers of 256 columns
//   warps 2..5  epilogue: tcgen05.ld TMEM -> registers -> (bias / accumulate /
//               convert) -> global; overlaps the next tile's main loop
//
// Every wait is bounded (see common.cuh): on a timeout the CTA records a
// status and falls through to the TMEM release.
//
// The tile loop is factored so that the fused collective kernels can reuse it
// with a different tile order or an epilogue that stores to peer memory.
#pragma once

#include "common.cuh"

namespace dd {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int ACC_STAGES = 2;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int TMEM_COLS = ACC_STAGES * BN;  // 512
constexpr int NUM_THREADS = 192;
constexpr int NUM_EPI_THREADS = 128;
// 1024 B slack for manual alignment + tiles + barriers.
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + 256;

enum Flags : int {
  F_OUT_F32 = 1,      // D is fp32 (else bf16)
  F_ACCUMULATE = 2,   // D += result (else D = result)
  F_BIAS = 4,         // add bias[n] (bf16)
  F_BIAS_F32 = 8,     // bias is fp32
  F_TMA_EPI = 16,     // CTA-pair kernels: the tile leaves through shared memory + TMA (set by the host)
};

struct Params {
  int M, N, K, batch;
  void* D;
  long long ldd;       // elements
  long long strideD;   // elements between batches
  const void* bias;
  int flags;
  int group_m;         // tile-order grouping (rows of tiles swept per column sweep)
  StatusRecord* status;
};

struct SharedStorage {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[ACC_STAGES];
  uint64_t tmem_empty[ACC_STAGES];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm,
                                            int& tn, int& tb) {
  const int per_batch = tiles_m * tiles_n;
  tb = tile / per_batch;
  int t = tile - tb * per_batch;
  // grouped ordering: sweep group_m tile-rows for each tile-column, so that a
  // wave of CTAs shares A rows and B columns in L2.
  const int group_size = group_m * tiles_n;
  const int g = t / group_size;
  const int first_m = g * group_m;
  const int rows = min(group_m, tiles_m - first_m);
  const int r = t - g * group_size;
  tm = first_m + (r % rows);
  tn = r / rows;
}

// Stores one 32-column chunk of one output row.
__device__ __forceinline__ void store_chunk(const Params& p, uint32_t (&acc)[32], long long row_off,
                                            int col0, int ncols_valid, bool vec_ok) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]);
  if (p.flags & F_BIAS) {
    if (p.flags & F_BIAS_F32) {
      const float* b = reinterpret_cast<const float*>(p.bias) + col0;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncols_valid) v[i] += __ldg(b + i);
    } else {
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < ncols_valid) v[i] += __bfloat162float(__ldg(b + i));
    }
  }
  if (p.flags & F_OUT_F32) {
    float* d = reinterpret_cast<float*>(p.D) + row_off + col0;
    if (vec_ok && ncols_valid == 32) {
      float4* d4 = reinterpret_cast<float4*>(d);
      if (p.flags & F_ACCUMULATE) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float4 o = d4[i];
          v[4 * i] += o.x; v[4 * i + 1] += o.y; v[4 * i + 2] += o.z; v[4 * i + 3] += o.w;
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) d4[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
      for (int i = 0; i < ncols_valid; ++i) d[i] = (p.flags & F_ACCUMULATE) ? d[i] + v[i] : v[i];
    }
  } else {
    __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.D) + row_off + col0;
    if (vec_ok && ncols_valid == 32) {
      uint4* d4 = reinterpret_cast<uint4*>(d);
      if (p.flags & F_ACCUMULATE) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 o = d4[i];
          float2 a = unpack_bf16x2(o.x), b = unpack_bf16x2(o.y), c = unpack_bf16x2(o.z), e = unpack_bf16x2(o.w);
          v[8 * i] += a.x; v[8 * i + 1] += a.y; v[8 * i + 2] += b.x; v[8 * i + 3] += b.y;
          v[8 * i + 4] += c.x; v[8 * i + 5] += c.y; v[8 * i + 6] += e.x; v[8 * i + 7] += e.y;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 o;
        o.x = pack_bf16x2(v[8 * i], v[8 * i + 1]);
        o.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
        o.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
        o.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
        d4[i] = o;
      }
    } else {
      for (int i = 0; i < ncols_valid; ++i) {
        float o = (p.flags & F_ACCUMULATE) ? __bfloat162float(d[i]) + v[i] : v[i];
        d[i] = __float2bfloat16(o);
      }
    }
  }
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles must sit on 1024 B boundaries.
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedStorage* ss = reinterpret_cast<SharedStorage*>(tiles + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n * p.batch;
  const int num_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ss->full[s], 1);
      mbar_init(&ss->empty[s], 1);
    }
    for (int a = 0; a < ACC_STAGES; ++a) {
      mbar_init(&ss->tmem_full[a], 1);
      mbar_init(&ss->tmem_empty[a], NUM_EPI_THREADS / 32);
    }
    ss->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ss->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn, tb;
        tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn, tb);
        for (int k = 0; k < num_k; ++k) {
          ok = mbar_wait(&ss->empty[stage], phase ^ 1, &ss->abort_flag, p.status, 1);
          if (!ok) break;
          uint8_t* sa = tiles + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&ss->full[stage], STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(sa + j * (64 * BK * 2), &tmap_a, &ss->full[stage], tm * BM + j * 64, k * BK, tb);
          } else {
            tma_load_3d(sa, &tmap_a, &ss->full[stage], k * BK, tm * BM, tb);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (64 * BK * 2), &tmap_b, &ss->full[stage], tn * BN + j * 64, k * BK, tb);
          } else {
            tma_load_3d(sb, &tmap_b, &ss->full[stage], k * BK, tn * BN, tb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // On an abort some loads may still be in flight towards this CTA's
      // shared memory: give them a bounded time to land before leaving.
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        ok = mbar_wait(&ss->tmem_empty[acc], acc_phase ^ 1, &ss->abort_flag, p.status, 2);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int k = 0; k < num_k; ++k) {
          ok = mbar_wait(&ss->full[stage], phase, &ss->abort_flag, p.status, 3);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // K-major: 16 k-elements = 32 B inside the 128 B swizzled row.
            // MN-major: 16 k-rows of 128 B = 2048 B.
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_f16(tmem_d, adesc, bdesc, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&ss->empty[stage]);  // frees the smem stage when the MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&ss->tmem_full[acc]);  // accumulator complete
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    // A warp may only touch the TMEM lane quarter given by (warp id % 4).
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = ((p.flags & F_OUT_F32) ? (p.ldd % 4 == 0) : (p.ldd % 8 == 0)) &&
                        ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) &&
                        ((p.strideD % 8) == 0);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn, tb;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn, tb);
      ok = mbar_wait(&ss->tmem_full[acc], acc_phase, &ss->abort_flag, p.status, 4);
      if (!ok) break;
      tc_fence_after();
      const int row = tm * BM + quarter * 32 + lane;
      const long long row_off = (long long)tb * p.strideD + (long long)row * p.ldd;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row < p.M) store_chunk(p, r, row_off, col0, min(32, p.N - col0), vec_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ss->tmem_empty[acc]);
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm
}  // namespace dd
