// Flash attention backward for sm_100a on tcgen05 + TMEM + TMA.
//
// Three launches:
//   1. delta[b,h,s] = sum_d O * dO                       (elementwise, fp32)
//   2. dK/dV kernel: one CTA per (kv tile j, kv head, batch) sweeps the query
//      tiles i >= j of every query head of the group:
//          S = Q_i K_j^T, dP = dO_i V_j^T           (TMEM)
//          P = exp(S*scale - lse), dS = P (dP - delta) scale   (softmax warps,
//          bf16 tiles in 128B-swizzled shared memory, row = query)
//          dV_j += P^T dO_i, dK_j += dS^T Q_i        (TMEM accumulators; the P /
//          dS tiles are fed as MN-major A operands, the Q / dO tiles that TMA
//          brought in K-major are re-read as MN-major B operands: same bytes)
//   3. dQ kernel: one CTA per (query tile i, head, batch) sweeps kv tiles j <= i,
//      recomputes S and dP, and accumulates dQ_i += dS K_j in TMEM.
// Recomputing S/dP in (3) costs two extra MMAs per tile pair and avoids global
// atomics, so the result is deterministic.
//
// Every wait is bounded; a timeout records a status and the CTA falls through
// to its TMEM release.  Sequence length must be a multiple of 128.
#include "common.cuh"
#include "runtime.cuh"

using namespace dd;

namespace {

constexpr int BT = 128;  // tile edge for queries and keys
constexpr int NUM_THREADS = 320;      // TMA warp, MMA warp, two softmax warpgroups (column halves)
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  const float* lse;     // [batch][Hq][S]
  const float* delta;   // [batch][Hq][S]
  __nv_bfloat16* dq; long long dq_row, dq_head;
  __nv_bfloat16* dk; long long dk_row, dk_head;
  __nv_bfloat16* dv; long long dv_row, dv_head;
  int S, Hq, Hkv, batch, causal;
  float scale;
  StatusRecord* status;
};

// One softmax-thread step shared by both kernels: reads row `row` of S and dP
// from TMEM, forms P and dS (bf16) and stores them into the swizzled tiles.
// sP may be null (dQ kernel needs only dS).
// `half` selects the 64 key columns this thread handles: P and dS need no row-wide
// reduction in the backward pass (lse and delta are given), so the two softmax
// warpgroups split every row between them.
__device__ __forceinline__ void form_p_ds(uint32_t tS, uint32_t tdP, uint8_t* sP, uint8_t* sdS, int row,
                                          float lse_l2, float delta, float c, float scale, bool diag, int half) {
  // all four tensor-memory loads of this thread's 64 columns are in flight before the first use
  uint32_t s[2][32], dp[2][32];
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    tmem_ld_32x32(tS + (2 * half + q) * 32, s[q]);
    tmem_ld_32x32(tdP + (2 * half + q) * 32, dp[q]);
  }
  tmem_ld_wait();
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int ch = 2 * half + q;
    uint32_t pp[16], pds[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float p0 = exp2f(__uint_as_float(s[q][i]) * c - lse_l2);
      float p1 = exp2f(__uint_as_float(s[q][i + 1]) * c - lse_l2);
      if (diag) {
        if (ch * 32 + i > row) p0 = 0.f;
        if (ch * 32 + i + 1 > row) p1 = 0.f;
      }
      const float d0 = p0 * (__uint_as_float(dp[q][i]) - delta) * scale;
      const float d1 = p1 * (__uint_as_float(dp[q][i + 1]) - delta) * scale;
      pp[i >> 1] = pack_bf16x2(p0, p1);
      pds[i >> 1] = pack_bf16x2(d0, d1);
    }
    const int off = (ch >> 1) * (BT * 128) + row * 128;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int grp = ((ch & 1) * 4 + g) ^ (row & 7);
      if (sP != nullptr)
        *reinterpret_cast<uint4*>(sP + off + (grp << 4)) =
            make_uint4(pp[4 * g], pp[4 * g + 1], pp[4 * g + 2], pp[4 * g + 3]);
      *reinterpret_cast<uint4*>(sdS + off + (grp << 4)) =
          make_uint4(pds[4 * g], pds[4 * g + 1], pds[4 * g + 2], pds[4 * g + 3]);
    }
  }
}

// Writes one TMEM accumulator row (D fp32) as bf16 to `dst`.
template <int D>
__device__ __forceinline__ void store_acc_row(uint32_t taddr, __nv_bfloat16* dst, bool valid) {
#pragma unroll 1
  for (int ch = 0; ch < D / 32; ++ch) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + ch * 32, r);
    tmem_ld_wait();
    if (valid) {
      uint4* d4 = reinterpret_cast<uint4*>(dst + ch * 32);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(r[8 * g]), __uint_as_float(r[8 * g + 1]));
        v.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]), __uint_as_float(r[8 * g + 3]));
        v.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]), __uint_as_float(r[8 * g + 5]));
        v.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]), __uint_as_float(r[8 * g + 7]));
        d4[g] = v;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// delta = rowsum(O * dO); one warp per (token, head) row.
// ---------------------------------------------------------------------------
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                  float* __restrict__ delta, int batch, int S, int Hq, int D) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long rows = (long long)batch * S * Hq;
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* o = O + row * D;
  const __nv_bfloat16* g = dO + row * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(o + i));
    const float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(g + i));
    acc += a.x * b.x + a.y * b.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const long long t = row / Hq;
    const int h = (int)(row - t * Hq);
    const long long b = t / S;
    const int s = (int)(t - b * S);
    delta[(b * Hq + h) * S + s] = acc;
  }
}

// ---------------------------------------------------------------------------
// dK / dV kernel
// ---------------------------------------------------------------------------
template <int D>
struct KVSmem {
  static constexpr int T_BYTES = BT * D * 2;        // one [128 x D] tile
  static constexpr int P_BYTES = BT * BT * 2;
  static constexpr int TILE_BYTES = 4 * T_BYTES + 2 * P_BYTES;
  static constexpr int TOTAL = 1024 + TILE_BYTES + 256;
};

struct KVBarriers {
  uint64_t kv_full, q_full, q_empty, do_full, do_empty, sdp_full, sdp_empty, pds_full, pds_empty, acc_done;
  uint32_t tmem_base;
  volatile int abort_flag;
};

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                     const BwdParams p) {
  using SM = KVSmem<D>;
  constexpr int DCH = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = tiles;
  uint8_t* sV = sK + SM::T_BYTES;
  uint8_t* sQ = sV + SM::T_BYTES;
  uint8_t* sdO = sQ + SM::T_BYTES;
  uint8_t* sP = sdO + SM::T_BYTES;
  uint8_t* sdS = sP + SM::P_BYTES;
  KVBarriers* bar = reinterpret_cast<KVBarriers*>(tiles + SM::TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nT = p.S / BT;
  const int G = p.Hq / p.Hkv;
  // small j (long sweeps) first
  const int id = blockIdx.x;
  const int j = id / (p.Hkv * p.batch);
  const int hb = id % (p.Hkv * p.batch);
  const int hkv = hb % p.Hkv, b = hb / p.Hkv;
  const int i0 = p.causal ? j : 0;
  const int iters = G * (nT - i0);
  const int kv_row0 = b * p.S + j * BT;

  if (threadIdx.x == 0) {
    mbar_init(&bar->kv_full, 1);
    mbar_init(&bar->q_full, 1); mbar_init(&bar->q_empty, 1);
    mbar_init(&bar->do_full, 1); mbar_init(&bar->do_empty, 1);
    mbar_init(&bar->sdp_full, 1); mbar_init(&bar->sdp_empty, 8);
    mbar_init(&bar->pds_full, 8); mbar_init(&bar->pds_empty, 1);
    mbar_init(&bar->acc_done, 1);
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bar->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 256 + D;

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v); tma_prefetch_desc(&tmap_do);
      mbar_expect_tx(&bar->kv_full, 2 * SM::T_BYTES);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_3d(sK + c * (BT * 128), &tmap_k, &bar->kv_full, c * 64, kv_row0, hkv);
        tma_load_3d(sV + c * (BT * 128), &tmap_v, &bar->kv_full, c * 64, kv_row0, hkv);
      }
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int h = hkv * G + it / (nT - i0);
        const int i = i0 + it % (nT - i0);
        const int q_row0 = b * p.S + i * BT;
        const uint32_t ph = it & 1;
        ok = mbar_wait(&bar->q_empty, ph ^ 1, &bar->abort_flag, p.status, 31);
        if (!ok) break;
        mbar_expect_tx(&bar->q_full, SM::T_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c) tma_load_3d(sQ + c * (BT * 128), &tmap_q, &bar->q_full, c * 64, q_row0, h);
        ok = mbar_wait(&bar->do_empty, ph ^ 1, &bar->abort_flag, p.status, 32);
        if (!ok) break;
        mbar_expect_tx(&bar->do_full, SM::T_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c) tma_load_3d(sdO + c * (BT * 128), &tmap_do, &bar->do_full, c * 64, q_row0, h);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BT, BT, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc_bf16(BT, D, 1, 1);  // A = P / dS (MN-major), B = dO / Q (MN-major)
      bool ok = mbar_wait(&bar->kv_full, 0, &bar->abort_flag, p.status, 33);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO),
                     aP = smem_u32(sP), adS = smem_u32(sdS);
      for (int it = 0; it < iters && ok; ++it) {
        const uint32_t ph = it & 1;
        ok = mbar_wait(&bar->sdp_empty, ph ^ 1, &bar->abort_flag, p.status, 34);
        if (!ok) break;
        ok = mbar_wait(&bar->q_full, ph, &bar->abort_flag, p.status, 35);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BT * 128) + (kk % 4) * 32;
          umma_f16(tS, make_smem_desc_sw128(aQ + off, 16, 1024), make_smem_desc_sw128(aK + off, 16, 1024),
                   idesc_s, kk > 0 ? 1u : 0u);
        }
        ok = mbar_wait(&bar->do_full, ph, &bar->abort_flag, p.status, 36);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BT * 128) + (kk % 4) * 32;
          umma_f16(tdP, make_smem_desc_sw128(adO + off, 16, 1024), make_smem_desc_sw128(aV + off, 16, 1024),
                   idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bar->sdp_full);
        ok = mbar_wait(&bar->pds_full, ph, &bar->abort_flag, p.status, 37);
        if (!ok) break;
        tc_fence_after();
        // contraction over the 128 queries: 8 steps of 16 query rows (2048 B)
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk) {
          const uint32_t off = kk * (16 * 128);
          umma_f16(tdV, make_smem_desc_sw128(aP + off, BT * 128, 1024), make_smem_desc_sw128(adO + off, BT * 128, 1024),
                   idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bar->do_empty);
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk) {
          const uint32_t off = kk * (16 * 128);
          umma_f16(tdK, make_smem_desc_sw128(adS + off, BT * 128, 1024), make_smem_desc_sw128(aQ + off, BT * 128, 1024),
                   idesc_acc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bar->q_empty);
        umma_commit(&bar->pds_empty);
      }
      if (ok) umma_commit(&bar->acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;               // softmax warpgroup = column half
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const float c = p.scale * kLog2e;
    bool ok = true;
    for (int it = 0; it < iters && ok; ++it) {
      const int h = hkv * G + it / (nT - i0);
      const int i = i0 + it % (nT - i0);
      const uint32_t ph = it & 1;
      const size_t stat = ((size_t)b * p.Hq + h) * p.S + i * BT + row;
      const float lse_l2 = __ldg(p.lse + stat) * kLog2e;
      const float delta = __ldg(p.delta + stat);
      ok = mbar_wait(&bar->sdp_full, ph, &bar->abort_flag, p.status, 38);
      if (!ok) break;
      ok = mbar_wait(&bar->pds_empty, ph ^ 1, &bar->abort_flag, p.status, 39);
      if (!ok) break;
      tc_fence_after();
      form_p_ds(tS + lane_off, tdP + lane_off, sP, sdS, row, lse_l2, delta, c, p.scale, p.causal && i == j, half);
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) { mbar_arrive(&bar->sdp_empty); mbar_arrive(&bar->pds_full); }
    }
    if (ok) ok = mbar_wait(&bar->acc_done, 0, &bar->abort_flag, p.status, 40);
    if (ok) {
      tc_fence_after();
      const long long t = kv_row0 + row;
      if (half == 0) store_acc_row<D>(tdV + lane_off, p.dv + t * p.dv_row + (long long)hkv * p.dv_head, true);
      else           store_acc_row<D>(tdK + lane_off, p.dk + t * p.dk_row + (long long)hkv * p.dk_head, true);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------
// dQ kernel
// ---------------------------------------------------------------------------
constexpr int DQ_STAGES = 2;
template <int D>
struct QSmem {
  static constexpr int T_BYTES = BT * D * 2;
  static constexpr int P_BYTES = BT * BT * 2;
  static constexpr int TILE_BYTES = 2 * T_BYTES + 2 * DQ_STAGES * T_BYTES + P_BYTES;
  static constexpr int TOTAL = 1024 + TILE_BYTES + 256;
};
struct QBarriers {
  uint64_t qdo_full;
  uint64_t k_full[DQ_STAGES], k_empty[DQ_STAGES], v_full[DQ_STAGES], v_empty[DQ_STAGES];
  uint64_t sdp_full, sdp_empty, ds_full, ds_empty, acc_done;
  uint32_t tmem_base;
  volatile int abort_flag;
};

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                   const BwdParams p) {
  using SM = QSmem<D>;
  constexpr int DCH = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = tiles;
  uint8_t* sdO = sQ + SM::T_BYTES;
  uint8_t* sK = sdO + SM::T_BYTES;
  uint8_t* sV = sK + DQ_STAGES * SM::T_BYTES;
  uint8_t* sdS = sV + DQ_STAGES * SM::T_BYTES;
  QBarriers* bar = reinterpret_cast<QBarriers*>(tiles + SM::TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nT = p.S / BT;
  const int id = blockIdx.x;
  const int hb = id % (p.Hq * p.batch);
  const int i = nT - 1 - id / (p.Hq * p.batch);
  const int h = hb % p.Hq, b = hb / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int nblocks = p.causal ? i + 1 : nT;
  const int q_row0 = b * p.S + i * BT;
  const int kv_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(&bar->qdo_full, 1);
    for (int s = 0; s < DQ_STAGES; ++s) {
      mbar_init(&bar->k_full[s], 1); mbar_init(&bar->k_empty[s], 1);
      mbar_init(&bar->v_full[s], 1); mbar_init(&bar->v_empty[s], 1);
    }
    mbar_init(&bar->sdp_full, 1); mbar_init(&bar->sdp_empty, 8);
    mbar_init(&bar->ds_full, 8); mbar_init(&bar->ds_empty, 1);
    mbar_init(&bar->acc_done, 1);
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bar->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;
  const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdQ = tmem_base + 256;

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v); tma_prefetch_desc(&tmap_do);
      mbar_expect_tx(&bar->qdo_full, 2 * SM::T_BYTES);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_3d(sQ + c * (BT * 128), &tmap_q, &bar->qdo_full, c * 64, q_row0, h);
        tma_load_3d(sdO + c * (BT * 128), &tmap_do, &bar->qdo_full, c * 64, q_row0, h);
      }
      bool ok = true;
      for (int jj = 0; jj < nblocks && ok; ++jj) {
        const int st = jj % DQ_STAGES;
        const uint32_t ph = (jj / DQ_STAGES) & 1;
        ok = mbar_wait(&bar->k_empty[st], ph ^ 1, &bar->abort_flag, p.status, 51);
        if (!ok) break;
        mbar_expect_tx(&bar->k_full[st], SM::T_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sK + st * SM::T_BYTES + c * (BT * 128), &tmap_k, &bar->k_full[st], c * 64, kv_base + jj * BT, hkv);
        ok = mbar_wait(&bar->v_empty[st], ph ^ 1, &bar->abort_flag, p.status, 52);
        if (!ok) break;
        mbar_expect_tx(&bar->v_full[st], SM::T_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sV + st * SM::T_BYTES + c * (BT * 128), &tmap_v, &bar->v_full[st], c * 64, kv_base + jj * BT, hkv);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BT, BT, 0, 0);
      constexpr uint32_t idesc_dq = make_idesc_bf16(BT, D, 0, 1);  // A = dS K-major, B = K_j MN-major
      bool ok = mbar_wait(&bar->qdo_full, 0, &bar->abort_flag, p.status, 53);
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), adS = smem_u32(sdS);
      for (int jj = 0; jj < nblocks && ok; ++jj) {
        const int st = jj % DQ_STAGES;
        const uint32_t ph = (jj / DQ_STAGES) & 1;
        const uint32_t aK = smem_u32(sK + st * SM::T_BYTES), aV = smem_u32(sV + st * SM::T_BYTES);
        ok = mbar_wait(&bar->sdp_empty, (jj & 1) ^ 1, &bar->abort_flag, p.status, 54);
        if (!ok) break;
        ok = mbar_wait(&bar->k_full[st], ph, &bar->abort_flag, p.status, 55);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BT * 128) + (kk % 4) * 32;
          umma_f16(tS, make_smem_desc_sw128(aQ + off, 16, 1024), make_smem_desc_sw128(aK + off, 16, 1024),
                   idesc_s, kk > 0 ? 1u : 0u);
        }
        ok = mbar_wait(&bar->v_full[st], ph, &bar->abort_flag, p.status, 56);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BT * 128) + (kk % 4) * 32;
          umma_f16(tdP, make_smem_desc_sw128(adO + off, 16, 1024), make_smem_desc_sw128(aV + off, 16, 1024),
                   idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bar->v_empty[st]);
        umma_commit(&bar->sdp_full);
        ok = mbar_wait(&bar->ds_full, jj & 1, &bar->abort_flag, p.status, 57);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk) {
          const uint32_t aoff = (kk / 4) * (BT * 128) + (kk % 4) * 32;   // dS: K-major over kv
          const uint32_t boff = kk * (16 * 128);                          // K_j: 16 kv rows
          umma_f16(tdQ, make_smem_desc_sw128(adS + aoff, 16, 1024), make_smem_desc_sw128(aK + boff, BT * 128, 1024),
                   idesc_dq, (jj > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bar->k_empty[st]);
        umma_commit(&bar->ds_empty);
      }
      if (ok) umma_commit(&bar->acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;               // softmax warpgroup = column half
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const float c = p.scale * kLog2e;
    const size_t stat = ((size_t)b * p.Hq + h) * p.S + i * BT + row;
    const float lse_l2 = __ldg(p.lse + stat) * kLog2e;
    const float delta = __ldg(p.delta + stat);
    bool ok = true;
    for (int jj = 0; jj < nblocks && ok; ++jj) {
      ok = mbar_wait(&bar->sdp_full, jj & 1, &bar->abort_flag, p.status, 58);
      if (!ok) break;
      ok = mbar_wait(&bar->ds_empty, (jj & 1) ^ 1, &bar->abort_flag, p.status, 59);
      if (!ok) break;
      tc_fence_after();
      form_p_ds(tS + lane_off, tdP + lane_off, nullptr, sdS, row, lse_l2, delta, c, p.scale, p.causal && jj == i, half);
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) { mbar_arrive(&bar->sdp_empty); mbar_arrive(&bar->ds_full); }
    }
    if (ok) ok = mbar_wait(&bar->acc_done, 0, &bar->abort_flag, p.status, 60);
    if (ok) {
      tc_fence_after();
      const long long t = q_row0 + row;
      store_acc_row<D / 2>(tdQ + lane_off + half * (D / 2), p.dq + t * p.dq_row + (long long)h * p.dq_head + half * (D / 2),
                           true);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int D>
int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
               const BwdParams& p, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto k1 = attn_bwd_dkdv_kernel<D>;
  auto k2 = attn_bwd_dq_kernel<D>;
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, KVSmem<D>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, QSmem<D>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  const int nT = p.S / BT;
  k1<<<nT * p.Hkv * p.batch, NUM_THREADS, KVSmem<D>::TOTAL, stream>>>(tq, tk, tv, tdo, p);
  k2<<<nT * p.Hq * p.batch, NUM_THREADS, QSmem<D>::TOTAL, stream>>>(tq, tk, tv, tdo, p);
  return (int)cudaGetLastError();
}

}  // namespace

// out / dout: contiguous [tokens][Hq][D]; delta: scratch [batch][Hq][S] fp32.
DD_API int dd_attn_bwd(const void* q, long long q_row, long long q_head, const void* k, long long k_row,
                       long long k_head, const void* v, long long v_row, long long v_head, const void* out,
                       const void* dout, const float* lse, float* delta, void* dq, long long dq_row,
                       long long dq_head, void* dk, long long dk_row, long long dk_head, void* dv, long long dv_row,
                       long long dv_head, int batch, int S, int Hq, int Hkv, int D, int causal, float scale,
                       void* stream) {
  if (S % 128 != 0 || (D != 64 && D != 128) || Hq % Hkv != 0 || batch <= 0) return DD_ERR_BAD_ARG;
  if ((dq_row | dq_head | dk_row | dk_head | dv_row | dv_head) % 8) return DD_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv)) & 15)
    return DD_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const uint64_t tokens = (uint64_t)batch * S;
  const long long rows = (long long)tokens * Hq;
  attn_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(out),
                                                             reinterpret_cast<const __nv_bfloat16*>(dout), delta,
                                                             batch, S, Hq, D);
  CUtensorMap tq, tk, tv, tdo;
  int r = get_tensor_map_bf16_3d(&tq, q, D, tokens, Hq, q_row * 2, q_head * 2, 64, BT);
  if (r) return r;
  r = get_tensor_map_bf16_3d(&tk, k, D, tokens, Hkv, k_row * 2, k_head * 2, 64, BT);
  if (r) return r;
  r = get_tensor_map_bf16_3d(&tv, v, D, tokens, Hkv, v_row * 2, v_head * 2, 64, BT);
  if (r) return r;
  r = get_tensor_map_bf16_3d(&tdo, dout, D, tokens, Hq, (uint64_t)Hq * D * 2, (uint64_t)D * 2, 64, BT);
  if (r) return r;
  int err = 0;
  BwdParams p;
  p.lse = lse; p.delta = delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq); p.dq_row = dq_row; p.dq_head = dq_head;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk); p.dk_row = dk_row; p.dk_head = dk_head;
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv); p.dv_row = dv_row; p.dv_head = dv_head;
  p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.batch = batch; p.causal = causal; p.scale = scale;
  p.status = device_status(&err);
  if (err) return err;
  return D == 128 ? launch_bwd<128>(tq, tk, tv, tdo, p, s) : launch_bwd<64>(tq, tk, tv, tdo, p, s);
}
