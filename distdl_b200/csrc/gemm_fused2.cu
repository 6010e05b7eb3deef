// CTA-pair (tcgen05 cta_group::2) versions of the fused all-gather -> GEMM and
// GEMM -> reduce-scatter kernels.  Protocols, flags and geometry are those of
// gemm_fused.cu; the difference is the tile: a pair of CTAs computes 256 rows x
// 256 columns, CTA r of the pair taking the row-block with order index
// 2 * tile_m + r (row-blocks of one pair need not be adjacent in memory: each CTA
// loads, accumulates and stores its own 128 rows, only the B slices are shared).
#include "gemm2_tcgen05.cuh"
#include "gemm_fused_common.cuh"
#include "runtime.cuh"

using namespace dd;
using namespace dd::fused;
namespace g2 = dd::gemm2;

namespace {

constexpr int PAIR_FUSED_THREADS = g2::NUM_THREADS + 128;

// MODE 1 = ag_gemm (AgParams), MODE 2 = gemm_rs (RsParams)
template <bool B_MN, int MODE, typename FP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MODE == 1 ? PAIR_FUSED_THREADS : g2::NUM_THREADS, 1)
fused_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ RsOutMaps omaps, const FP fp) {
  const Params& p = fp.g;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = tiles + g2::STAGES * g2::STAGE_BYTES;
  g2::SharedStorage* ss = reinterpret_cast<g2::SharedStorage*>(out_stage + g2::OUT_STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = g2::cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const Geometry geo = fp.geo;
  const int row_blocks = geo.row_blocks();
  const int tiles_m = (row_blocks + 1) / 2;
  const int tiles_n = (p.N + g2::BN - 1) / g2::BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_k = (p.K + g2::BK - 1) / g2::BK;
  // ag_gemm: own shard first; gemm_rs: remote owners first
  const int first = (MODE == 1) ? geo.me : (geo.me + 1) % geo.P;

  if (threadIdx.x == 0) {
    for (int s = 0; s < g2::STAGES; ++s) { mbar_init(&ss->full[s], 1); mbar_init(&ss->empty[s], 1); }
    for (int a = 0; a < g2::ACC_STAGES; ++a) { mbar_init(&ss->tmem_full[a], 1); mbar_init(&ss->tmem_empty[a], 8); }
    ss->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { g2::tmem_alloc_pair(&ss->tmem_base, g2::TMEM_COLS); g2::tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  g2::cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = ss->tmem_base;

  if (MODE == 1 && warp >= 6) {
    // ------------------------------ comm warps (ag_gemm) ------------------------------
    if constexpr (MODE == 1) {
      const int ct = threadIdx.x - g2::NUM_THREADS;
      if (blockIdx.x == 0 && ct < geo.P && ct != geo.me) red_release_sys(fp.pad[ct] + PAD_AG + fp.writer[geo.me]);
      bool ok = true;
      const size_t row_bytes = (size_t)p.K * 2;
      const size_t piece_vecs = (size_t)(BM / kPullSub) * row_bytes / 16;
      bool peers_checked = false;
      // pieces are numbered block-major in tile order (own shard first), so the
      // first wave of CTAs stages what the first tiles need
      const int pieces = row_blocks * kPullSub;
      for (int u = blockIdx.x; u < pieces && ok; u += gridDim.x) {
        const int o = u / kPullSub, sub = u - o * kPullSub;
        int owner, lb;
        const int rb = geo.block_of(o, geo.me, owner, lb);
        if (owner != geo.me && !peers_checked) {
          if (ct < geo.P && ct != geo.me)
            wait_counter<true>(fp.pad[geo.me] + PAD_AG + fp.writer[ct], fp.expect[ct], &ss->abort_flag, p.status, 231);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          peers_checked = true;
          ok = ss->abort_flag == 0;
          if (!ok) break;
        }
        const size_t piece_off = ((size_t)sub * (BM / kPullSub)) * row_bytes;
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(fp.shard[owner]) +
                                                          (size_t)lb * BM * row_bytes + piece_off);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(fp.G) + (size_t)rb * BM * row_bytes + piece_off);
        size_t v = ct;
        for (; v + 7 * 128 < piece_vecs; v += 8 * 128) {
          uint4 r[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) r[q] = ld_peer16(src + v + q * 128);
#pragma unroll
          for (int q = 0; q < 8; ++q) dst[v + q * 128] = r[q];
        }
        for (; v < piece_vecs; v += 128) dst[v] = ld_peer16(src + v);
        __threadfence();
        proxy_fence_global();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ct == 0) {
          const uint32_t old = atom_add_acq_rel_gpu(fp.ready_cnt + rb, 1u);
          if (old == kPullSub - 1) {
            fp.ready_cnt[rb] = 0;
            st_release_gpu(fp.ready + rb, fp.epoch);
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ct == 0) {
        __threadfence();
        const uint32_t old = atomicAdd(fp.done_counter, 1u);
        if (old + 1 == fp.done_target) {
          __threadfence_system();
          for (int i = 0; i < geo.P; ++i)
            if (i != geo.me) red_release_sys(fp.pad[i] + PAD_AG + fp.writer[geo.me]);
        }
      }
      if (blockIdx.x == 0 && ct < geo.P && ct != geo.me)
        wait_counter<true>(fp.pad[geo.me] + PAD_AG + fp.writer[ct], fp.end_expect[ct], &ss->abort_flag, p.status, 232);
    }
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int last_ready = -1;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn, tb;
        gemm::tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn, tb);
        const int o = 2 * tm + (int)rank;
        int owner = 0, lb = 0;
        // a missing second block (odd count) loads rows past the end: TMA fills zeros
        const int rb = o < row_blocks ? geo.block_of(o, first, owner, lb) : row_blocks;
        if (MODE == 1 && o < row_blocks && rb != last_ready) {
          if constexpr (MODE == 1) {
            ok = wait_counter<false>(fp.ready + rb, fp.epoch, &ss->abort_flag, p.status, 233);
            if (!ok) break;
            proxy_fence_global();
          }
          last_ready = rb;
        }
        const int n0 = tn * g2::BN + (int)rank * g2::BNH;
        for (int k = 0; k < num_k; ++k) {
          ok = mbar_wait(&ss->empty[stage], phase ^ 1, &ss->abort_flag, p.status, 301);
          if (!ok) break;
          uint8_t* sa = tiles + stage * g2::STAGE_BYTES;
          uint8_t* sb = sa + g2::A_STAGE_BYTES;
          const uint32_t full_leader = g2::mapa(smem_u32(&ss->full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&ss->full[stage], 2 * g2::STAGE_BYTES);
          g2::tma_load_3d_pair(sa, &tmap_a, full_leader, k * g2::BK, rb * BM, 0);
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < g2::BNH / 64; ++j)
              g2::tma_load_3d_pair(sb + j * (64 * g2::BK * 2), &tmap_b, full_leader, n0 + j * 64, k * g2::BK, 0);
          } else {
            g2::tma_load_3d_pair(sb, &tmap_b, full_leader, k * g2::BK, n0, 0);
          }
          if (++stage == g2::STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * g2::BM, g2::BN, 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        ok = mbar_wait(&ss->tmem_empty[acc], acc_phase ^ 1, &ss->abort_flag, p.status, 302);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * g2::BN;
        for (int k = 0; k < num_k; ++k) {
          ok = mbar_wait(&ss->full[stage], phase, &ss->abort_flag, p.status, 303);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(tiles + stage * g2::STAGE_BYTES);
          const uint32_t sb = sa + g2::A_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < g2::BK / g2::UMMA_K; ++kk) {
            const uint64_t adesc = make_smem_desc_sw128(sa + kk * (g2::UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (g2::UMMA_K * 128), 64 * g2::BK * 2, 1024)
                                        : make_smem_desc_sw128(sb + kk * (g2::UMMA_K * 2), 16, 1024);
            g2::umma_f16_pair(tmem_d, adesc, bdesc, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          g2::umma_commit_pair(&ss->empty[stage]);
          if (++stage == g2::STAGES) { stage = 0; phase ^= 1; }
        }
        g2::umma_commit_pair(&ss->tmem_full[acc]);
        if (++acc == g2::ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    Params q = p;
    bool vec_ok;
    if constexpr (MODE == 2) {
      if (et < geo.P && et != geo.me)
        wait_counter<true>(fp.pad[geo.me] + PAD_RS_CONSUMED + fp.parity * 8 + fp.writer[et], fp.consumed_expect[et],
                           &ss->abort_flag, p.status, 241);
      asm volatile("bar.sync 2, 128;" ::: "memory");
      ok = ss->abort_flag == 0;
      q.flags = p.flags & (F_BIAS | F_BIAS_F32);
      q.ldd = p.N;
      vec_ok = (p.N % 8 == 0);
    } else {
      vec_ok = ((p.flags & F_OUT_F32) ? (p.ldd % 4 == 0) : (p.ldd % 8 == 0)) &&
               ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0);
    }
    // gemm_rs with the fold inside: once this CTA's tiles for the other members are stored
    // (they come first), it reports "delivered" and, before its first own tile, waits for
    // the partials of the peers
    bool delivered_sent = false;
    const __nv_bfloat16* addends[kMaxPeers];
    int n_add = 0;
    auto signal_delivered = [&]() {
      if constexpr (MODE == 2) {
        if (fp.tma_store && lane == 0) {
          tma_store_wait_all();
          proxy_fence_global();
        }
        __threadfence_system();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (et == 0) {
          const uint32_t old = atomicAdd(fp.done_counter, 1u);
          if (old + 1 == fp.done_target) {
            __threadfence_system();
            for (int i = 0; i < geo.P; ++i)
              if (i != geo.me) red_release_sys(fp.pad[i] + PAD_RS_DELIVERED + fp.parity * 8 + fp.writer[geo.me]);
          }
        }
        delivered_sent = true;
      }
    };
    if constexpr (MODE == 2) {
      if (fp.fold)
        for (int i = 0; i < geo.P; ++i)
          if (i != geo.me) addends[n_add++] = fp.my_slot[i];
    }
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int tm, tn, tb;
      gemm::tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn, tb);
      const int o = 2 * tm + (int)rank;
      int owner = 0, lb = 0;
      const int rb = o < row_blocks ? geo.block_of(o, first, owner, lb) : row_blocks;
      bool own = false;
      if constexpr (MODE == 2) {
        own = fp.fold && owner == geo.me && o < row_blocks;
        if (own && !delivered_sent) {
          signal_delivered();
          if (et < geo.P && et != geo.me)
            wait_counter<true>(fp.pad[geo.me] + PAD_RS_DELIVERED + fp.parity * 8 + fp.writer[et],
                               fp.delivered_expect[et], &ss->abort_flag, p.status, 221);
          asm volatile("bar.sync 2, 128;" ::: "memory");
          ok = ss->abort_flag == 0;
          if (!ok) break;
        }
      }
      ok = mbar_wait(&ss->tmem_full[acc], acc_phase, &ss->abort_flag, p.status, 304);
      if (!ok) break;
      tc_fence_after();
      long long row_off;
      if constexpr (MODE == 2) {
        q.D = fp.slot[owner];
        row_off = ((long long)lb * BM + quarter * 32 + lane) * p.N;
      } else {
        row_off = ((long long)rb * BM + quarter * 32 + lane) * p.ldd;
      }
      const uint32_t taddr = tmem_base + acc * g2::BN + ((uint32_t)(quarter * 32) << 16);
      // TMA epilogue: omaps.m[owner] is the owner's slot (gemm_rs) / omaps.m[0] is D (ag_gemm)
      bool stored;
      if constexpr (MODE == 2) stored = fp.tma_store != 0;
      else stored = (p.flags & F_TMA_EPI) != 0;
      if (stored) {
        if constexpr (MODE == 2) {
          g2::epilogue_tma(q, &omaps.m[owner], taddr, out_stage + quarter * g2::OUT_WARP_BYTES, lane, tn * g2::BN,
                           lb * BM + quarter * 32, 0, o < row_blocks, addends, own ? n_add : 0, (long long)p.N);
        } else {
          g2::epilogue_tma(q, &omaps.m[0], taddr, out_stage + quarter * g2::OUT_WARP_BYTES, lane, tn * g2::BN,
                           rb * BM + quarter * 32, 0, o < row_blocks);
        }
      }
#pragma unroll 1
      for (int c = 0; c < g2::BN / 32 && !stored; ++c) {
        const int col0 = tn * g2::BN + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (o < row_blocks) store_chunk(q, r, row_off, col0, min(32, p.N - col0), vec_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) g2::mbar_arrive_cluster(g2::mapa(smem_u32(&ss->tmem_empty[acc]), 0));
      if (++acc == g2::ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
    if constexpr (MODE == 1) {
      if ((p.flags & F_TMA_EPI) && lane == 0) tma_store_wait_all();
    }
    if constexpr (MODE == 2) {
      if (!fp.fold) {
        signal_delivered();
      } else {
        if (!delivered_sent) signal_delivered();      // a CTA without own tiles
        // all own tiles written: the peers may reuse my staging slots of this parity
        if (fp.tma_store && lane == 0) tma_store_wait_all();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (et == 0) {
          __threadfence();
          const uint32_t old = atomicAdd(fp.done_counter2, 1u);
          if (old + 1 == fp.done_target2) {
            __threadfence_system();
            for (int i = 0; i < geo.P; ++i)
              if (i != geo.me) red_release_sys(fp.pad[i] + PAD_RS_CONSUMED + fp.parity * 8 + fp.writer[geo.me]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  g2::cluster_sync();
  if (warp == 1) { tc_fence_after(); g2::tmem_dealloc_pair(tmem_base, g2::TMEM_COLS); }
}

template <typename K>
int set_smem(K kern) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, g2::SMEM_BYTES);
}

}  // namespace

// Launchers used by gemm_fused.cu when CTA pairs are enabled.  The tensor maps
// must have been encoded with the pair tile boxes (A: {64, 128}; B: {64, 128}
// K-major or {64, 64} MN-major).
int dd_launch_ag_pair(const CUtensorMap& ta, const CUtensorMap& tb, const RsOutMaps& om, const AgParams& ap, int w_mn,
                      int ctas, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    int r;
    if ((r = set_smem(fused_pair_kernel<false, 1, AgParams>))) return r;
    if ((r = set_smem(fused_pair_kernel<true, 1, AgParams>))) return r;
    configured = true;
  }
  if (w_mn) fused_pair_kernel<true, 1, AgParams><<<ctas, PAIR_FUSED_THREADS, g2::SMEM_BYTES, s>>>(ta, tb, om, ap);
  else      fused_pair_kernel<false, 1, AgParams><<<ctas, PAIR_FUSED_THREADS, g2::SMEM_BYTES, s>>>(ta, tb, om, ap);
  return (int)cudaGetLastError();
}

int dd_launch_rs_pair(const CUtensorMap& ta, const CUtensorMap& tb, const RsOutMaps& om, const RsParams& rp, int w_mn,
                      int ctas, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    int r;
    if ((r = set_smem(fused_pair_kernel<false, 2, RsParams>))) return r;
    if ((r = set_smem(fused_pair_kernel<true, 2, RsParams>))) return r;
    configured = true;
  }
  if (w_mn) fused_pair_kernel<true, 2, RsParams><<<ctas, g2::NUM_THREADS, g2::SMEM_BYTES, s>>>(ta, tb, om, rp);
  else      fused_pair_kernel<false, 2, RsParams><<<ctas, g2::NUM_THREADS, g2::SMEM_BYTES, s>>>(ta, tb, om, rp);
  return (int)cudaGetLastError();
}
