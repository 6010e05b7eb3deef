// Fused compute + collective GEMMs for tensor parallelism with sequence
// sharding, over peer-mapped memory (NVLink / NVSwitch).  Same tcgen05 / TMEM /
// TMA pipeline as gemm_tcgen05.cuh; the collective runs inside the kernel.
//
// Geometry shared by both kernels.  A logical activation [batch, seq, feat] is
// split along `seq` over the P members of a team: member r holds
// [batch, seq/P, feat].  Row-block = 128 consecutive rows of the flattened
// [batch*seq, feat] matrix; seq/P is a multiple of 128, so a row-block belongs
// to exactly one member.
//
// ag_gemm   (all-gather -> GEMM):   D[batch*seq, N] = gather(X)[.., K] * W[N, K]^T
//   Four extra "comm" warps per CTA pull the peers' shards (plain 16-byte peer
//   loads) into the local gathered buffer G, one row-block at a time, and
//   publish a per-row-block ready word; the TMA producer of whichever CTA needs
//   that row-block waits for the word (bounded) before it loads A tiles from G.
//   TMA only ever reads local memory.  Row-blocks are fetched, and tiles are
//   scheduled, local shard first, so the first remote hop hides behind compute.
//   G stays valid after the kernel (the weight-gradient GEMM needs it).
//
// gemm_rs   (GEMM -> reduce-scatter): each member computes the full
//   [batch*seq, N] partial product; the epilogue stores every tile straight into
//   the staging slot [source = me] of the member that owns those rows (peer
//   stores for remote owners, scheduled first so that they overlap the remaining
//   tiles).  When its last CTA has finished, a member raises "delivered" on every
//   peer.  rs_reduce_kernel (a second launch) waits for all "delivered" words,
//   sums the P slots in fp32, writes the bf16 result and raises
//   "consumed" on the peers, which the next gemm_rs using the same staging
//   parity waits for before it overwrites the slot.
//
//
// This file holds the host entry points, the single-CTA-tile kernels (fallback,
// `DISTDL_FUSED_PAIR=0`) and the separate fold kernel.  The default kernels are the
// CTA-pair versions in gemm_fused2.cu; they differ in three ways: row blocks are
// pulled in 32-row pieces spread over all CTAs (the shard staging is double buffered,
// so a kernel waits for the readers of the PREVIOUS call only), tiles leave through
// shared memory and TMA stores (also into a peer's slot), and gemm_rs folds the
// partials inside the GEMM: a CTA reports "delivered" once its tiles for the other
// members are stored, and its tiles of this member's own rows, which come last, add
// the partials the peers delivered and go straight to the output.
//
// All flags are counters that only grow; every wait is bounded (2 s) and
// reports through the status record; once a wait has run out, later waits fail at
// once.
#include <cstdlib>
#include <cstring>

#include "gemm_fused_common.cuh"
#include "runtime.cuh"

using namespace dd;
using namespace dd::gemm;
using namespace dd::fused;

namespace {

template <bool B_MN>
__global__ void __launch_bounds__(FUSED_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const AgParams ap) {
  const Params& p = ap.g;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedStorage* ss = reinterpret_cast<SharedStorage*>(tiles + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = ap.geo.row_blocks();
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ss->full[s], 1); mbar_init(&ss->empty[s], 1); }
    for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(&ss->tmem_full[a], 1); mbar_init(&ss->tmem_empty[a], NUM_EPI_THREADS / 32); }
    ss->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&ss->tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss->tmem_base;

  if (warp >= 6) {
    // ------------------------------ comm warps ------------------------------
    const int ct = threadIdx.x - NUM_THREADS;        // 0..127
    const Geometry geo = ap.geo;
    // tell the peers that my shard is staged (stream order put the copy before this kernel)
    if (blockIdx.x == 0 && ct < geo.P && ct != geo.me)
      red_release_sys(ap.pad[ct] + PAD_AG + ap.writer[geo.me]);
    bool ok = true;
    const size_t row_bytes = (size_t)p.K * 2;
    const size_t block_vecs = (size_t)BM * row_bytes / 16;
    bool peers_checked = false;
    for (int o = blockIdx.x; o < tiles_m && ok; o += gridDim.x) {
      int owner, lb;
      const int rb = geo.block_of(o, geo.me, owner, lb);
      if (owner != geo.me && !peers_checked) {
        // first remote block of this CTA: all peers must have staged their shards
        if (ct < geo.P && ct != geo.me)
          wait_counter<true>(ap.pad[geo.me] + PAD_AG + ap.writer[ct], ap.expect[ct], &ss->abort_flag, p.status, 201);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        peers_checked = true;
        ok = ss->abort_flag == 0;
        if (!ok) break;
      }
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(ap.shard[owner]) +
                                                        (size_t)lb * BM * row_bytes);
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(ap.G) + (size_t)rb * BM * row_bytes);
      size_t v = ct;
      for (; v + 7 * 128 < block_vecs; v += 8 * 128) {
        uint4 r[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) r[u] = ld_peer16(src + v + u * 128);
#pragma unroll
        for (int u = 0; u < 8; ++u) dst[v + u * 128] = r[u];
      }
      for (; v < block_vecs; v += 128) dst[v] = ld_peer16(src + v);
      __threadfence();
      proxy_fence_global();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ct == 0) st_release_gpu(ap.ready + rb, ap.epoch);
    }
    // this CTA is done pulling: the last CTA of the GPU tells the peers
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (ct == 0) {
      __threadfence();
      const uint32_t old = atomicAdd(ap.done_counter, 1u);
      if (old + 1 == ap.done_target) {
        __threadfence_system();
        for (int i = 0; i < geo.P; ++i)
          if (i != geo.me) red_release_sys(ap.pad[i] + PAD_AG + ap.writer[geo.me]);
      }
    }
    // my shard may only be overwritten once every peer has pulled it
    if (blockIdx.x == 0 && ct < geo.P && ct != geo.me)
      wait_counter<true>(ap.pad[geo.me] + PAD_AG + ap.writer[ct], ap.end_expect[ct], &ss->abort_flag, p.status, 202);
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int last_ready = -1;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int to, tn, tb;
        tile_coords(tile, tiles_m, tiles_n, p.group_m, to, tn, tb);
        int owner, lb;
        const int rb = ap.geo.block_of(to, ap.geo.me, owner, lb);
        if (rb != last_ready) {
          ok = wait_counter<false>(ap.ready + rb, ap.epoch, &ss->abort_flag, p.status, 203);
          if (!ok) break;
          proxy_fence_global();
          last_ready = rb;
        }
        for (int k = 0; k < num_k; ++k) {
          ok = mbar_wait(&ss->empty[stage], phase ^ 1, &ss->abort_flag, p.status, 1);
          if (!ok) break;
          uint8_t* sa = tiles + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&ss->full[stage], STAGE_BYTES);
          tma_load_3d(sa, &tmap_a, &ss->full[stage], k * BK, rb * BM, 0);
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (64 * BK * 2), &tmap_b, &ss->full[stage], tn * BN + j * 64, k * BK, 0);
          } else {
            tma_load_3d(sb, &tmap_b, &ss->full[stage], k * BK, tn * BN, 0);
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
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
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
            const uint64_t adesc = make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_f16(tmem_d, adesc, bdesc, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&ss->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&ss->tmem_full[acc]);
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool vec_ok = ((p.flags & F_OUT_F32) ? (p.ldd % 4 == 0) : (p.ldd % 8 == 0)) &&
                        ((reinterpret_cast<uintptr_t>(p.D) & 15) == 0);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int to, tn, tb;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, to, tn, tb);
      int owner, lb;
      const int rb = ap.geo.block_of(to, ap.geo.me, owner, lb);
      ok = mbar_wait(&ss->tmem_full[acc], acc_phase, &ss->abort_flag, p.status, 4);
      if (!ok) break;
      tc_fence_after();
      const int row = rb * BM + quarter * 32 + lane;
      const long long row_off = (long long)row * p.ldd;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) break;
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
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// ------------------------------- gemm_rs -----------------------------------
template <bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const RsParams rp) {
  const Params& p = rp.g;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  SharedStorage* ss = reinterpret_cast<SharedStorage*>(tiles + STAGES * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = rp.geo.row_blocks();
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_k = (p.K + BK - 1) / BK;
  // remote owners first: their stores cross NVLink while the local tiles compute
  const int first = (rp.geo.me + 1) % rp.geo.P;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ss->full[s], 1); mbar_init(&ss->empty[s], 1); }
    for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(&ss->tmem_full[a], 1); mbar_init(&ss->tmem_empty[a], NUM_EPI_THREADS / 32); }
    ss->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&ss->tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ss->tmem_base;

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int to, tn, tb;
        tile_coords(tile, tiles_m, tiles_n, p.group_m, to, tn, tb);
        int owner, lb;
        const int rb = rp.geo.block_of(to, first, owner, lb);
        for (int k = 0; k < num_k; ++k) {
          ok = mbar_wait(&ss->empty[stage], phase ^ 1, &ss->abort_flag, p.status, 1);
          if (!ok) break;
          uint8_t* sa = tiles + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&ss->full[stage], STAGE_BYTES);
          tma_load_3d(sa, &tmap_a, &ss->full[stage], k * BK, rb * BM, 0);
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (64 * BK * 2), &tmap_b, &ss->full[stage], tn * BN + j * 64, k * BK, 0);
          } else {
            tma_load_3d(sb, &tmap_b, &ss->full[stage], k * BK, tn * BN, 0);
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
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
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
            const uint64_t adesc = make_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sb + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                        : make_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
            umma_f16(tmem_d, adesc, bdesc, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&ss->empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        umma_commit(&ss->tmem_full[acc]);
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;                  // 0..127 inside the epilogue group
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // the slots on the peers are free once they consumed the previous use of this parity
    if (et < rp.geo.P && et != rp.geo.me)
      wait_counter<true>(rp.pad[rp.geo.me] + PAD_RS_CONSUMED + rp.parity * 8 + rp.writer[et], rp.consumed_expect[et],
                         &ss->abort_flag, p.status, 211);
    asm volatile("bar.sync 2, 128;" ::: "memory");
    ok = ss->abort_flag == 0;
    Params q = p;                                     // per-tile destination
    q.flags = p.flags & (F_BIAS | F_BIAS_F32);        // bf16, overwrite; a member that holds the bias adds it to
    q.ldd = p.N;                                      // its partial product, so it enters the sum exactly once
    const bool vec_ok = (p.N % 8 == 0);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int to, tn, tb;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, to, tn, tb);
      int owner, lb;
      rp.geo.block_of(to, first, owner, lb);
      ok = mbar_wait(&ss->tmem_full[acc], acc_phase, &ss->abort_flag, p.status, 4);
      if (!ok) break;
      tc_fence_after();
      q.D = rp.slot[owner];
      const long long row_off = ((long long)lb * BM + quarter * 32 + lane) * p.N;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = tn * BN + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        store_chunk(q, r, row_off, col0, min(32, p.N - col0), vec_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ss->tmem_empty[acc]);
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
    // all stores of this CTA are out: count it; the last CTA raises "delivered"
    __threadfence_system();
    asm volatile("bar.sync 2, 128;" ::: "memory");
    if (et == 0) {
      const uint32_t old = atomicAdd(rp.done_counter, 1u);
      if (old + 1 == rp.done_target) {
        __threadfence_system();
        for (int i = 0; i < rp.geo.P; ++i)
          if (i != rp.geo.me) red_release_sys(rp.pad[i] + PAD_RS_DELIVERED + rp.parity * 8 + rp.writer[rp.geo.me]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

// out[rows, N] = sum_src staging[src][rows, N] (+ bias); waits for "delivered".
struct ReduceParams {
  int P, me, parity;
  const __nv_bfloat16* staging;      // local staging base: [P][rows][N]
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;
  long long rows;
  int N;
  uint32_t* pad[kMaxPeers];
  int writer[kMaxPeers];
  uint32_t delivered_expect[kMaxPeers];
  uint32_t* done_counter;
  uint32_t done_target;
  StatusRecord* status;
};

__global__ void __launch_bounds__(256) rs_reduce_kernel(const ReduceParams rp) {
  __shared__ int abort_flag;
  if (threadIdx.x == 0) abort_flag = 0;
  __syncthreads();
  if (threadIdx.x < rp.P && threadIdx.x != rp.me)
    wait_counter<true>(rp.pad[rp.me] + PAD_RS_DELIVERED + rp.parity * 8 + rp.writer[threadIdx.x],
                       rp.delivered_expect[threadIdx.x], &abort_flag, rp.status, 221);
  __syncthreads();
  if (abort_flag) return;
  const long long slot_elems = rp.rows * rp.N;
  const long long nvec = slot_elems >> 3;
  const int nv_row = rp.N >> 3;
  // kRedUnroll independent vectors per thread and iteration keep enough loads in
  // flight to cover the HBM latency
  constexpr int kRedUnroll = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * kRedUnroll) {
    uint4 u[kRedUnroll][kMaxPeers];
#pragma unroll
    for (int q = 0; q < kRedUnroll; ++q) {
      const long long v = v0 + q * stride;
      if (v < nvec) {
#pragma unroll
        for (int s = 0; s < kMaxPeers; ++s)
          if (s < rp.P) u[q][s] = ld_peer16(rp.staging + (long long)s * slot_elems + v * 8);
      }
    }
#pragma unroll
    for (int q = 0; q < kRedUnroll; ++q) {
      const long long v = v0 + q * stride;
      if (v >= nvec) break;
      float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s) {
        if (s < rp.P) {
          float2 f;
          f = unpack_bf16x2(u[q][s].x); a[0] += f.x; a[1] += f.y;
          f = unpack_bf16x2(u[q][s].y); a[2] += f.x; a[3] += f.y;
          f = unpack_bf16x2(u[q][s].z); a[4] += f.x; a[5] += f.y;
          f = unpack_bf16x2(u[q][s].w); a[6] += f.x; a[7] += f.y;
        }
      }
      if (rp.bias != nullptr) {
        const int c = (int)(v % nv_row) * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] += __bfloat162float(rp.bias[c + j]);
      }
      uint4 o = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]),
                           pack_bf16x2(a[6], a[7]));
      *reinterpret_cast<uint4*>(rp.out + v * 8) = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t old = atomicAdd(rp.done_counter, 1u);
    if (old + 1 == rp.done_target) {
      __threadfence_system();
      for (int i = 0; i < rp.P; ++i)
        if (i != rp.me) red_release_sys(rp.pad[i] + PAD_RS_CONSUMED + rp.parity * 8 + rp.writer[rp.me]);
    }
  }
}

template <typename K>
int set_smem(K kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace

DD_API int dd_fused_reduce_ctas() { return kReduceCtas; }

static bool fused_pair_enabled() {
  static const bool on = []() { const char* e = getenv("DISTDL_FUSED_PAIR"); return !(e && e[0] == '0'); }();
  return on;
}
// Grid size of the fused GEMM kernels (the completion counters count CTAs).
DD_API int dd_fused_gemm_ctas() { return fused_pair_enabled() ? (current_sm_count() & ~1) : current_sm_count(); }

// All pointer arrays have P entries in team order.  `w` is the [N, K] weight
// (w_mn = 0) or its [K, N] storage read as MN-major (w_mn = 1, ldw = N-stride).
DD_API int dd_ag_gemm(int P, int me, void* const* shards, void* G, const void* w, int w_mn, long long ldw, void* D,
                      long long ldd, const void* bias, int bias_f32, int batch, int s_local, int N, int K,
                      void* ready, unsigned epoch, void* const* pads, const int* writers, const unsigned* expect,
                      void* done_counter, unsigned done_target, int max_ctas, void* ready_cnt,
                      const unsigned* end_expect, void* stream) {
  if (P < 1 || P > kMaxPeers || s_local % BM || K % 8 || ldw % 8) return DD_ERR_BAD_ARG;
  const long long M = (long long)batch * P * s_local;
  CUtensorMap ta, tb;
  int r = get_tensor_map_bf16_3d(&ta, G, K, M, 1, (uint64_t)K * 2, (uint64_t)M * K * 2, BK, BM);
  if (r) return r;
  const bool pair = fused_pair_enabled();
  if (w_mn) r = get_tensor_map_bf16_3d(&tb, w, N, K, 1, ldw * 2, (uint64_t)K * ldw * 2, 64, BK);
  else      r = get_tensor_map_bf16_3d(&tb, w, K, N, 1, ldw * 2, (uint64_t)N * ldw * 2, BK, pair ? 128 : BN);
  if (r) return r;
  int err = 0;
  AgParams ap;
  ap.g.M = (int)M; ap.g.N = N; ap.g.K = K; ap.g.batch = 1;
  ap.g.D = D; ap.g.ldd = ldd; ap.g.strideD = M * ldd;
  ap.g.bias = bias; ap.g.flags = bias ? (F_BIAS | (bias_f32 ? F_BIAS_F32 : 0)) : 0;
  ap.g.group_m = 8;
  ap.g.status = device_status(&err);
  if (err) return err;
  ap.geo.P = P; ap.geo.me = me; ap.geo.batch = batch; ap.geo.s_local = s_local;
  for (int i = 0; i < P; ++i) {
    ap.shard[i] = shards[i];
    ap.pad[i] = reinterpret_cast<uint32_t*>(pads[i]);
    ap.writer[i] = writers[i];
    ap.expect[i] = expect[i];
    ap.end_expect[i] = end_expect ? end_expect[i] : expect[i] + 1;
  }
  ap.ready_cnt = reinterpret_cast<uint32_t*>(ready_cnt);
  ap.G = reinterpret_cast<__nv_bfloat16*>(G);
  ap.ready = reinterpret_cast<uint32_t*>(ready);
  ap.epoch = epoch;
  ap.done_counter = reinterpret_cast<uint32_t*>(done_counter);
  ap.done_target = done_target;
  int ctas = dd_fused_gemm_ctas();
  if (pair) {
    if (ready_cnt == nullptr) return DD_ERR_BAD_ARG;
    ap.g.group_m = 4;
    static const bool tma_epi = []() { const char* e = getenv("DISTDL_GEMM_TMA_EPI"); return !(e && e[0] == '0'); }();
    RsOutMaps om;
    memset(&om, 0, sizeof(om));
    if (tma_epi && (reinterpret_cast<uintptr_t>(D) & 15) == 0 && ldd % 8 == 0) {
      r = get_tensor_map_bf16_3d(&om.m[0], D, N, M, 1, (uint64_t)ldd * 2, (uint64_t)M * ldd * 2, 64, 32);
      if (r) return r;
      ap.g.flags |= F_TMA_EPI;
    }
    return dd_launch_ag_pair(ta, tb, om, ap, w_mn, ctas, reinterpret_cast<cudaStream_t>(stream));
  }
  static bool configured = false;
  if (!configured) {
    if ((r = set_smem(ag_gemm_kernel<false>, SMEM_BYTES))) return r;
    if ((r = set_smem(ag_gemm_kernel<true>, SMEM_BYTES))) return r;
    configured = true;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // every CTA takes part in the pull, so the grid is fixed (done_target counts CTAs)
  if (w_mn) ag_gemm_kernel<true><<<ctas, FUSED_THREADS, SMEM_BYTES, s>>>(ta, tb, ap);
  else      ag_gemm_kernel<false><<<ctas, FUSED_THREADS, SMEM_BYTES, s>>>(ta, tb, ap);
  return (int)cudaGetLastError();
}

// 1 when dd_gemm_rs folds the partials inside the GEMM kernel for this geometry (CTA pairs,
// TMA stores, and a member's row blocks a multiple of the 8-block tile group, so that every
// CTA meets all tiles of the other members before its own); the completion counter of the
// reduction then counts the GEMM's CTAs.
DD_API int dd_gemm_rs_folds(int batch, int s_local) {
  static const bool on = []() {
    const char* e = getenv("DISTDL_RS_FOLD");
    const char* t = getenv("DISTDL_RS_TMA_STORE");
    return !(e && e[0] == '0') && !(t && t[0] == '0');
  }();
  if (!on || !fused_pair_enabled() || s_local % BM) return 0;
  const long long blocks = (long long)batch * (s_local / BM);
  return blocks % 8 == 0 ? 1 : 0;
}

// Launches the GEMM with scatter epilogue, then the reduction.  `slots[i]` =
// member i's staging slot for source `me`; `staging` = my own staging
// ([P][batch*s_local][N]); x is the local [batch*P*s_local, K] operand.
DD_API int dd_gemm_rs(int P, int me, const void* x, long long ldx, const void* w, int w_mn, long long ldw,
                      void* const* slots, const void* staging, void* out, const void* bias, int batch, int s_local,
                      int N, int K, int parity, void* const* pads, const int* writers, const unsigned* consumed_expect,
                      const unsigned* delivered_expect, void* done_counter_gemm, unsigned done_target_gemm,
                      void* done_counter_reduce, unsigned done_target_reduce, int max_ctas, void* stream) {
  if (P < 1 || P > kMaxPeers || s_local % BM || K % 8 || ldw % 8 || ldx % 8 || N % 8) return DD_ERR_BAD_ARG;
  const long long M = (long long)batch * P * s_local;
  CUtensorMap ta, tb;
  int r = get_tensor_map_bf16_3d(&ta, x, K, M, 1, (uint64_t)ldx * 2, (uint64_t)M * ldx * 2, BK, BM);
  if (r) return r;
  const bool pair = fused_pair_enabled();
  if (w_mn) r = get_tensor_map_bf16_3d(&tb, w, N, K, 1, ldw * 2, (uint64_t)K * ldw * 2, 64, BK);
  else      r = get_tensor_map_bf16_3d(&tb, w, K, N, 1, ldw * 2, (uint64_t)N * ldw * 2, BK, pair ? 128 : BN);
  if (r) return r;
  int err = 0;
  RsParams rp;
  rp.g.M = (int)M; rp.g.N = N; rp.g.K = K; rp.g.batch = 1;
  rp.g.D = nullptr; rp.g.ldd = N; rp.g.strideD = 0; rp.g.bias = bias; rp.g.flags = bias ? F_BIAS : 0;
  rp.g.group_m = 8;
  rp.g.status = device_status(&err);
  if (err) return err;
  rp.geo.P = P; rp.geo.me = me; rp.geo.batch = batch; rp.geo.s_local = s_local;
  rp.parity = parity;
  for (int i = 0; i < P; ++i) {
    rp.slot[i] = reinterpret_cast<__nv_bfloat16*>(slots[i]);
    rp.pad[i] = reinterpret_cast<uint32_t*>(pads[i]);
    rp.writer[i] = writers[i];
    rp.consumed_expect[i] = consumed_expect[i];
  }
  rp.done_counter = reinterpret_cast<uint32_t*>(done_counter_gemm);
  rp.done_target = done_target_gemm;
  int ctas = dd_fused_gemm_ctas();
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  rp.tma_store = 0;
  rp.fold = 0;
  rp.done_counter2 = reinterpret_cast<uint32_t*>(done_counter_reduce);
  rp.done_target2 = done_target_reduce;
  bool fold = false;
  if (pair) {
    rp.g.group_m = 4;
    static const bool tma_store = []() { const char* e = getenv("DISTDL_RS_TMA_STORE"); return !(e && e[0] == '0'); }();
    RsOutMaps om;
    memset(&om, 0, sizeof(om));
    if (tma_store) {
      const uint64_t rows = (uint64_t)batch * s_local;
      fold = dd_gemm_rs_folds(batch, s_local) != 0;
      for (int i = 0; i < P; ++i) {
        // with the fold inside the GEMM the tiles of my own rows go straight to the output
        void* base = (fold && i == me) ? out : slots[i];
        r = get_tensor_map_bf16_3d(&om.m[i], base, N, rows, 1, (uint64_t)N * 2, rows * N * 2, 64, 32);
        if (r) return r;
      }
      rp.tma_store = 1;
      if (fold) {
        rp.fold = 1;
        for (int i = 0; i < P; ++i) {
          rp.my_slot[i] = reinterpret_cast<const __nv_bfloat16*>(staging) + (size_t)i * rows * N;
          rp.delivered_expect[i] = delivered_expect[i];
        }
      }
    }
    r = dd_launch_rs_pair(ta, tb, om, rp, w_mn, ctas, s);
  } else {
    static bool configured = false;
    if (!configured) {
      if ((r = set_smem(gemm_rs_kernel<false>, SMEM_BYTES))) return r;
      if ((r = set_smem(gemm_rs_kernel<true>, SMEM_BYTES))) return r;
      configured = true;
    }
    if (w_mn) gemm_rs_kernel<true><<<ctas, NUM_THREADS, SMEM_BYTES, s>>>(ta, tb, rp);
    else      gemm_rs_kernel<false><<<ctas, NUM_THREADS, SMEM_BYTES, s>>>(ta, tb, rp);
    r = (int)cudaGetLastError();
  }
  if (r) return r;
  if (fold) return 0;
  ReduceParams q;
  q.P = P; q.me = me; q.parity = parity;
  q.staging = reinterpret_cast<const __nv_bfloat16*>(staging);
  q.out = reinterpret_cast<__nv_bfloat16*>(out);
  q.bias = nullptr;
  q.rows = (long long)batch * s_local; q.N = N;
  for (int i = 0; i < P; ++i) {
    q.pad[i] = reinterpret_cast<uint32_t*>(pads[i]);
    q.writer[i] = writers[i];
    q.delivered_expect[i] = delivered_expect[i];
  }
  q.done_counter = reinterpret_cast<uint32_t*>(done_counter_reduce);
  q.done_target = done_target_reduce;
  q.status = rp.g.status;
  rs_reduce_kernel<<<kReduceCtas, 256, 0, s>>>(q);
  return (int)cudaGetLastError();
}
