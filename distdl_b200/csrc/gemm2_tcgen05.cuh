// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2.
//
// Two CTAs of a cluster (two neighbouring SMs) share one 256x256 output tile:
// CTA r owns rows [128 r, 128 r + 128) of the tile (its TMEM holds that half of
// the accumulator) and stages, per 64-deep k-block, its own 128x64 slice of A
// and HALF of the 256x64 slice of B (rows [128 r, 128 r + 128) of B).  The
// tensor core of each SM reads the two B halves from both CTAs' shared memory,
// so a CTA moves 32 KB per k-block through shared memory instead of 48 KB: with
// single-CTA tiles the 128x256 MMA is limited by shared-memory bandwidth (TMA
// writes plus operand reads), which the pair removes.
//
// Roles per CTA: warp 0 TMA producer (each CTA loads its own slices; both signal
// the LEADER's full barrier, no multicast), warp 1 MMA issuer (leader CTA only),
// warps 2..5 epilogue (each CTA drains its own TMEM half).  tcgen05.commit towards
// each CTA's barrier releases smem stages and publishes accumulators in both CTAs.
// All waits are bounded; TMEM is allocated / freed pairwise by warp 1 of both CTAs.
#pragma once

#include "gemm_tcgen05.cuh"

namespace dd {
namespace gemm2 {

using gemm::Params;
using gemm::store_chunk;

constexpr int BM = 128;          // rows per CTA (256 per pair)
constexpr int BN = 256;          // columns per pair
constexpr int BNH = 128;         // B rows staged per CTA
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int ACC_STAGES = 2;
constexpr int A_STAGE_BYTES = BM * BK * 2;    // 16 KB
constexpr int B_STAGE_BYTES = BNH * BK * 2;   // 16 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int TMEM_COLS = ACC_STAGES * BN;
constexpr int NUM_THREADS = 192;
// epilogue staging: per epilogue warp two boxes of [32 rows][128 B]
constexpr int OUT_WARP_BYTES = 2 * 32 * 128;
constexpr int OUT_STAGE_BYTES = 4 * OUT_WARP_BYTES;          // 32 KB
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + OUT_STAGE_BYTES + 256;

struct SharedStorage {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[ACC_STAGES];
  uint64_t tmem_empty[ACC_STAGES];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa(uint32_t local_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: data to this CTA's shared memory, completion
// bytes to the mbarrier at `mbar_cluster_addr` (the leader's).
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* m, uint32_t mbar_cluster_addr,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(mbar_cluster_addr), "r"(c0), "r"(c1),
      "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive, once all previously issued MMAs of the pair have completed, on the
// barrier at `bar`'s offset in BOTH CTAs: one commit per destination (the local
// barrier and the peer's, addressed through the cluster window).
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint32_t local = smem_u32(bar);
  const uint32_t a0 = mapa(local, 0), a1 = mapa(local, 1);
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(a0) : "memory");
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(a1) : "memory");
}


// TMA epilogue of one warp: its 32 rows x BN columns of the accumulator at `taddr`
// go registers -> 128B-swizzled shared memory -> TMA, so that the tile leaves the SM
// as full 128-byte lines (local memory or a peer's, behind NVLink).  bf16 output:
// rounds of 128 columns (two boxes of 64); fp32: rounds of 64 columns (two boxes of
// 32), stored or, with F_ACCUMULATE, added at L2 by a TMA reduction, which spares
// the read of D.  `map` has box {64 | 32 columns, 32 rows}; rows and columns past
// the tensor are clipped by the hardware.  `write` = false skips the stores.
// `add_src[0 .. n_add)`: optional bf16 matrices [rows][add_ld] (local memory) whose rows
// row0 .. row0 + 31 are added to the tile before it is written (partials of other GPUs).
__device__ __forceinline__ void epilogue_tma(const Params& q, const CUtensorMap* map, uint32_t taddr, uint8_t* stage_w,
                                             int lane, int col_tile0, int row0, int tb, bool write,
                                             const __nv_bfloat16* const* add_src = nullptr, int n_add = 0,
                                             long long add_ld = 0) {
  const bool f32 = (q.flags & gemm::F_OUT_F32) != 0;
  const bool add = (q.flags & gemm::F_ACCUMULATE) != 0;
  const int round_cols = f32 ? 64 : 128;
  const int box_cols = round_cols / 2;
#pragma unroll 1
  for (int rd = 0; rd < BN / round_cols; ++rd) {
    const int colr = col_tile0 + rd * round_cols;
    if (colr >= q.N) break;
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
#pragma unroll 1
    for (int cc = 0; cc < round_cols / 32; ++cc) {
      const int col0 = colr + cc * 32;
      uint32_t r[32];
      tmem_ld_32x32(taddr + rd * round_cols + cc * 32, r);
      tmem_ld_wait();
      if ((q.flags & gemm::F_BIAS) && col0 < q.N) {
        const int nv = min(32, q.N - col0);
        if (q.flags & gemm::F_BIAS_F32) {
          const float* bp = reinterpret_cast<const float*>(q.bias) + col0;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < nv) r[i] = __float_as_uint(__uint_as_float(r[i]) + __ldg(bp + i));
        } else {
          const __nv_bfloat16* bp = reinterpret_cast<const __nv_bfloat16*>(q.bias) + col0;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < nv) r[i] = __float_as_uint(__uint_as_float(r[i]) + __bfloat162float(__ldg(bp + i)));
        }
      }
      if (n_add > 0 && write) {
        for (int a = 0; a < n_add; ++a) {
          const __nv_bfloat16* src = add_src[a] + (long long)(row0 + lane) * add_ld + col0;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (col0 + 8 * g < q.N) {
              const uint4 u = *reinterpret_cast<const uint4*>(src + 8 * g);
              float2 f;
              f = unpack_bf16x2(u.x); r[8 * g] = __float_as_uint(__uint_as_float(r[8 * g]) + f.x);
              r[8 * g + 1] = __float_as_uint(__uint_as_float(r[8 * g + 1]) + f.y);
              f = unpack_bf16x2(u.y); r[8 * g + 2] = __float_as_uint(__uint_as_float(r[8 * g + 2]) + f.x);
              r[8 * g + 3] = __float_as_uint(__uint_as_float(r[8 * g + 3]) + f.y);
              f = unpack_bf16x2(u.z); r[8 * g + 4] = __float_as_uint(__uint_as_float(r[8 * g + 4]) + f.x);
              r[8 * g + 5] = __float_as_uint(__uint_as_float(r[8 * g + 5]) + f.y);
              f = unpack_bf16x2(u.w); r[8 * g + 6] = __float_as_uint(__uint_as_float(r[8 * g + 6]) + f.x);
              r[8 * g + 7] = __float_as_uint(__uint_as_float(r[8 * g + 7]) + f.y);
            }
          }
        }
      }
      if (f32) {
        uint8_t* rowp = stage_w + cc * (32 * 128) + lane * 128;      // box cc: 32 fp32 = 128 B per row
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<uint4*>(rowp + ((g ^ (lane & 7)) << 4)) = make_uint4(r[4 * g], r[4 * g + 1], r[4 * g + 2],
                                                                               r[4 * g + 3]);
      } else {
        uint8_t* rowp = stage_w + (cc >> 1) * (32 * 128) + lane * 128;  // box cc / 2: 64 bf16 = 128 B per row
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[8 * g]), __uint_as_float(r[8 * g + 1]));
          v.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]), __uint_as_float(r[8 * g + 3]));
          v.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]), __uint_as_float(r[8 * g + 5]));
          v.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]), __uint_as_float(r[8 * g + 7]));
          const int chunk = (cc & 1) * 4 + g;
          *reinterpret_cast<uint4*>(rowp + ((chunk ^ (lane & 7)) << 4)) = v;
        }
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && write) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int c0 = colr + j * box_cols;
        if (c0 >= q.N) break;
        if (add) tma_reduce_add_3d(map, stage_w + j * (32 * 128), c0, row0, tb);
        else     tma_store_3d(map, stage_w + j * (32 * 128), c0, row0, tb);
      }
      tma_store_commit();
    }
  }
}

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn,
                                                 int& tb) {
  gemm::tile_coords(tile, tiles_m, tiles_n, group_m, tm, tn, tb);
}

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_d, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = tiles + STAGES * STAGE_BYTES;
  SharedStorage* ss = reinterpret_cast<SharedStorage*>(out_stage + OUT_STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n * p.batch;
  const int num_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ss->full[s], 1); mbar_init(&ss->empty[s], 1); }
    for (int a = 0; a < ACC_STAGES; ++a) {
      mbar_init(&ss->tmem_full[a], 1);
      mbar_init(&ss->tmem_empty[a], 2 * (gemm::NUM_EPI_THREADS / 32));   // epilogue warps of both CTAs
    }
    ss->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc_pair(&ss->tmem_base, TMEM_COLS); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync();                                   // barriers of both CTAs are initialised
  tc_fence_after();
  const uint32_t tmem_base = ss->tmem_base;

  if (warp == 0) {
    // ------------------- TMA producer (both CTAs, own slices) -------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn, tb;
        pair_tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn, tb);
        const int m0 = tm * 2 * BM + (int)rank * BM;
        const int n0 = tn * BN + (int)rank * BNH;
        for (int k = 0; k < num_k; ++k) {
          ok = mbar_wait(&ss->empty[stage], phase ^ 1, &ss->abort_flag, p.status, 301);
          if (!ok) break;
          uint8_t* sa = tiles + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          const uint32_t full_leader = mapa(smem_u32(&ss->full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&ss->full[stage], 2 * STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d_pair(sa + j * (64 * BK * 2), &tmap_a, full_leader, m0 + j * 64, k * BK, tb);
          } else {
            tma_load_3d_pair(sa, &tmap_a, full_leader, k * BK, m0, tb);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j)
              tma_load_3d_pair(sb + j * (64 * BK * 2), &tmap_b, full_leader, n0 + j * 64, k * BK, tb);
          } else {
            tma_load_3d_pair(sb, &tmap_b, full_leader, k * BK, n0, tb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ---------------------------- MMA issuer (leader) ---------------------------
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        ok = mbar_wait(&ss->tmem_empty[acc], acc_phase ^ 1, &ss->abort_flag, p.status, 302);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int k = 0; k < num_k; ++k) {
          ok = mbar_wait(&ss->full[stage], phase, &ss->abort_flag, p.status, 303);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sa + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_f16_pair(tmem_d, adesc, bdesc, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(&ss->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit_pair(&ss->tmem_full[acc]);
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------ epilogue (both CTAs, own half) ----------------------
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = ((p.flags & gemm::F_OUT_F32) ? (p.ldd % 4 == 0) : (p.ldd % 8 == 0)) &&
                        ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0) && ((p.strideD % 8) == 0);
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int tm, tn, tb;
      pair_tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn, tb);
      ok = mbar_wait(&ss->tmem_full[acc], acc_phase, &ss->abort_flag, p.status, 304);
      if (!ok) break;
      tc_fence_after();
      const int row = tm * 2 * BM + (int)rank * BM + quarter * 32 + lane;
      const long long row_off = (long long)tb * p.strideD + (long long)row * p.ldd;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      if (p.flags & gemm::F_TMA_EPI) {
        epilogue_tma(p, &tmap_d, taddr, out_stage + quarter * OUT_WARP_BYTES, lane, tn * BN,
                     tm * 2 * BM + (int)rank * BM + quarter * 32, tb, true);
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = tn * BN + c * 32;
          if (col0 >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (row < p.M) store_chunk(p, r, row_off, col0, min(32, p.N - col0), vec_ok);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa(smem_u32(&ss->tmem_empty[acc]), 0));
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
    if ((p.flags & gemm::F_TMA_EPI) && lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();               // nobody leaves while the peer may still touch its barriers / TMEM
  if (warp == 1) { tc_fence_after(); tmem_dealloc_pair(tmem_base, TMEM_COLS); }
}

}  // namespace gemm2
}  // namespace dd
