// Flash attention backward for sm_100a (head dimension DD_HEAD_DIM = 128 or 64; this file is
// included once per head dimension by attention_bwd2.cu, inside namespace DD_BWD2_NS): the
// probabilities never leave tensor memory and the softmax arithmetic overlaps the tensor-core work.
//
// Same three launches and the same arithmetic as attention_bwd.cu (pre-pass, dK / dV kernel,
// dQ kernel; S and dP are recomputed in both kernels, nothing is accumulated with atomics, so
// the result is deterministic), but built differently:
//
//   * dK / dV kernel: the products are formed TRANSPOSED, S^T = K_j Q_i^T and dP^T = V_j dO_i^T
//     (key rows in the tensor-memory lanes, queries in the columns).  The softmax threads write
//     P^T and dS^T as bf16 over the fp32 values they came from, and the accumulating products
//     dV_j += P^T dO_i and dK_j += dS^T Q_i read them from tensor memory as their A operands:
//     no shared-memory round trip for P / dS.  The per-query statistics (log-sum-exp in base 2,
//     delta) arrive in shared memory with the Q tile.
//   * dQ kernel: S = Q_i K_j^T, dP = dO_i V_j^T with the queries in the lanes; dS goes back to
//     tensor memory over dP and feeds dQ_i += dS K_j as the A operand.  dP is double-buffered.
//   * The pipeline is split per product: S of the next tile pair is issued as soon as the
//     softmax threads have consumed S of this one (while they still work on dS), dP of the next
//     pair as soon as dS of this one is in place, so the tensor cores work during the softmax
//     arithmetic instead of waiting for it.
//   * Sixteen softmax warps (four per tensor-memory lane quarter, 32 columns each) instead of
//     eight; the factor `scale` of dS is applied once to the dK / dQ accumulators in the epilogue.
//
// Every wait is bounded; a time-out records a status and the CTA falls through to its
// tensor-memory release.  Sequence length must be a multiple of 128.
namespace DD_BWD2_NS {

constexpr int BT = 128;               // tile edge for queries and keys
constexpr int D = DD_HEAD_DIM;         // head dimension
constexpr int SOFTMAX_WARPS = 16;
constexpr int NUM_THREADS = 64 + SOFTMAX_WARPS * 32;   // TMA warp, MMA warp, softmax warps
constexpr float kLog2e = 1.4426950408889634f;
constexpr int T_BYTES = BT * D * 2;   // one [128 x D] bf16 tile
constexpr int DCH = D / 64;           // 64-element (128-byte) chunks per row

struct Bwd2Params {
  const float* lse2;    // [batch][Hq][S]  log-sum-exp of the scaled scores, in base 2
  const float* delta;   // [batch][Hq][S]  rowsum(O * dO)
  __nv_bfloat16* dq; long long dq_row, dq_head;
  __nv_bfloat16* dk; long long dk_row, dk_head;
  __nv_bfloat16* dv; long long dv_row, dv_head;
  int S, Hq, Hkv, batch, causal;
  float scale;
  StatusRecord* status;
};

// Untiled bulk copy global -> shared of this CTA (both addresses 16-byte aligned, size a
// multiple of 16 bytes), completion on an mbarrier.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// 32 fp32 accumulator columns of this thread's lane, times `mul`, as bf16 to dst[0, 32)
__device__ __forceinline__ void store_cols32(uint32_t taddr, __nv_bfloat16* dst, float mul) {
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint4 v;
    v.x = pack_bf16x2(__uint_as_float(r[8 * g]) * mul, __uint_as_float(r[8 * g + 1]) * mul);
    v.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * mul, __uint_as_float(r[8 * g + 3]) * mul);
    v.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * mul, __uint_as_float(r[8 * g + 5]) * mul);
    v.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * mul, __uint_as_float(r[8 * g + 7]) * mul);
    d4[g] = v;
  }
}

// D[128 x 128] = A[128 x 128] B[128 x 128]^T, both operands K-major tiles in shared memory
__device__ __forceinline__ void issue_kmajor(uint32_t tmem_d, uint32_t a_addr, uint32_t b_addr) {
  constexpr uint32_t idesc = make_idesc_bf16(BT, BT, 0, 0);
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const uint32_t off = (kk / 4) * (BT * 128) + (kk % 4) * 32;
    umma_f16(tmem_d, make_smem_desc_sw128(a_addr + off, 16, 1024), make_smem_desc_sw128(b_addr + off, 16, 1024), idesc,
             kk > 0 ? 1u : 0u);
  }
}

// D[128 x D] (+)= A[128 x 128] B[128 x D]: A = bf16 pairs in tensor memory (rows in the lanes; the
// 16 values of contraction step kk sit in the 8 columns at (kk / 2) * 32 + (kk % 2) * 8, where the
// softmax warp of that column group left them), B = a [128 rows x D] tile in shared memory whose
// rows are the contraction index (MN-major).
__device__ __forceinline__ void issue_from_tmem(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_addr, bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(BT, D, 0, 1);
#pragma unroll
  for (int kk = 0; kk < BT / 16; ++kk)
    umma_f16_ts(tmem_d, tmem_a + (kk >> 1) * 32 + (kk & 1) * 8,
                make_smem_desc_sw128(b_addr + kk * (16 * 128), BT * 128, 1024), idesc, (accumulate || kk > 0) ? 1u : 0u);
}

// ---------------------------------------------------------------------------
// pre-pass: delta = rowsum(O * dO), lse2 = lse * log2(e); one warp per (token, head) row.
// ---------------------------------------------------------------------------
__global__ void attn_prepass_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                    const float* __restrict__ lse, float* __restrict__ delta,
                                    float* __restrict__ lse2, int batch, int S, int Hq) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long rows = (long long)batch * S * Hq;
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float acc;
  if (D == 128) {
    const uint2 a = *reinterpret_cast<const uint2*>(O + row * D + lane * 4);
    const uint2 g = *reinterpret_cast<const uint2*>(dO + row * D + lane * 4);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y);
    acc = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
  } else {
    const float2 a0 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(O + row * D + lane * 2));
    const float2 g0 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dO + row * D + lane * 2));
    acc = a0.x * g0.x + a0.y * g0.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    const long long t = row / Hq;
    const int h = (int)(row - t * Hq);
    const long long b = t / S;
    const int s = (int)(t - b * S);
    const size_t o = ((size_t)b * Hq + h) * S + s;
    delta[o] = acc;
    lse2[o] = lse[o] * kLog2e;
  }
}

// ---------------------------------------------------------------------------
// dK / dV kernel: one CTA per (kv tile j, kv head, batch) sweeps the query tiles i >= j of
// every query head of the group.
// ---------------------------------------------------------------------------
struct KVSmem {
  static constexpr int TILE_BYTES = 6 * T_BYTES;          // K, V, Q x 2, dO x 2
  static constexpr int STAT_BYTES = 2 * 2 * BT * 4;       // (lse2, delta) x 2 stages
  static constexpr int TOTAL = 1024 + TILE_BYTES + STAT_BYTES + 256;
};
struct KVBarriers {
  uint64_t kv_full, q_full[2], q_empty[2], do_full[2], do_empty[2], s_full, p_full, dp_full, ds_full, acc_done;
  uint32_t tmem_base;
  volatile int abort_flag;
};

template <bool POLY>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd2_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                      const Bwd2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = tiles;
  uint8_t* sV = sK + T_BYTES;
  uint8_t* sQ = sV + T_BYTES;             // 2 stages
  uint8_t* sdO = sQ + 2 * T_BYTES;        // 2 stages
  float* stats = reinterpret_cast<float*>(tiles + KVSmem::TILE_BYTES);   // [stage][lse2 128 | delta 128]
  KVBarriers* bar = reinterpret_cast<KVBarriers*>(tiles + KVSmem::TILE_BYTES + KVSmem::STAT_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nT = p.S / BT;
  const int G = p.Hq / p.Hkv;
  // small j (long sweeps) first
  const int id = blockIdx.x;
  const int j = id / (p.Hkv * p.batch);
  const int hb = id % (p.Hkv * p.batch);
  const int hkv = hb % p.Hkv, b = hb / p.Hkv;
  const int i0 = p.causal ? j : 0;
  const int per_head = nT - i0;
  const int iters = G * per_head;
  const int kv_row0 = b * p.S + j * BT;

  if (threadIdx.x == 0) {
    mbar_init(&bar->kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar->q_full[s], 1); mbar_init(&bar->q_empty[s], 1);
      mbar_init(&bar->do_full[s], 1); mbar_init(&bar->do_empty[s], 1);
    }
    mbar_init(&bar->s_full, 1); mbar_init(&bar->p_full, SOFTMAX_WARPS);
    mbar_init(&bar->dp_full, 1); mbar_init(&bar->ds_full, SOFTMAX_WARPS);
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
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v); tma_prefetch_desc(&tmap_do);
      mbar_expect_tx(&bar->kv_full, 2 * T_BYTES);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_3d(sK + c * (BT * 128), &tmap_k, &bar->kv_full, c * 64, kv_row0, hkv);
        tma_load_3d(sV + c * (BT * 128), &tmap_v, &bar->kv_full, c * 64, kv_row0, hkv);
      }
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int h = hkv * G + it / per_head;
        const int i = i0 + it % per_head;
        const int q_row0 = b * p.S + i * BT;
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        ok = mbar_wait(&bar->q_empty[st], ph ^ 1, &bar->abort_flag, p.status, 131);
        if (!ok) break;
        mbar_expect_tx(&bar->q_full[st], T_BYTES + 2 * BT * 4);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sQ + st * T_BYTES + c * (BT * 128), &tmap_q, &bar->q_full[st], c * 64, q_row0, h);
        const size_t stat = ((size_t)b * p.Hq + h) * p.S + (size_t)i * BT;
        bulk_load(stats + st * 2 * BT, p.lse2 + stat, BT * 4, &bar->q_full[st]);
        bulk_load(stats + st * 2 * BT + BT, p.delta + stat, BT * 4, &bar->q_full[st]);
        ok = mbar_wait(&bar->do_empty[st], ph ^ 1, &bar->abort_flag, p.status, 132);
        if (!ok) break;
        mbar_expect_tx(&bar->do_full[st], T_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sdO + st * T_BYTES + c * (BT * 128), &tmap_do, &bar->do_full[st], c * 64, q_row0, h);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (elect_one()) {
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), adO = smem_u32(sdO);
      bool ok = mbar_wait(&bar->kv_full, 0, &bar->abort_flag, p.status, 133);
      if (ok) ok = mbar_wait(&bar->q_full[0], 0, &bar->abort_flag, p.status, 134);
      if (ok) {
        tc_fence_after();
        issue_kmajor(tS, aK, aQ);                       // S^T(0)
        umma_commit(&bar->s_full);
        ok = mbar_wait(&bar->do_full[0], 0, &bar->abort_flag, p.status, 135);
      }
      if (ok) {
        tc_fence_after();
        issue_kmajor(tdP, aV, adO);                     // dP^T(0)
        umma_commit(&bar->dp_full);
      }
      for (int it = 0; it < iters && ok; ++it) {
        const int st = it & 1, nst = st ^ 1;
        const uint32_t nph = ((it + 1) >> 1) & 1;
        const bool more = it + 1 < iters;
        ok = mbar_wait(&bar->p_full, it & 1, &bar->abort_flag, p.status, 136);
        if (!ok) break;
        tc_fence_after();
        issue_from_tmem(tdV, tS, adO + st * T_BYTES, it > 0);         // dV += P^T dO
        umma_commit(&bar->do_empty[st]);
        if (more) {
          ok = mbar_wait(&bar->q_full[nst], nph, &bar->abort_flag, p.status, 137);
          if (!ok) break;
          tc_fence_after();
          issue_kmajor(tS, aK, aQ + nst * T_BYTES);                    // S^T(it + 1)
          umma_commit(&bar->s_full);
        }
        ok = mbar_wait(&bar->ds_full, it & 1, &bar->abort_flag, p.status, 138);
        if (!ok) break;
        tc_fence_after();
        issue_from_tmem(tdK, tdP, aQ + st * T_BYTES, it > 0);         // dK += dS^T Q
        umma_commit(&bar->q_empty[st]);
        if (more) {
          ok = mbar_wait(&bar->do_full[nst], nph, &bar->abort_flag, p.status, 139);
          if (!ok) break;
          tc_fence_after();
          issue_kmajor(tdP, aV, adO + nst * T_BYTES);                  // dP^T(it + 1)
          umma_commit(&bar->dp_full);
        }
      }
      if (ok) umma_commit(&bar->acc_done);
    }
  } else {
    // -------------------------------- softmax --------------------------------
    const int quarter = warp & 3;                   // tensor-memory lane quarter this warp may access
    const int cg = (warp - 2) >> 2;                 // 32-column group (queries) of this warp
    const int row = quarter * 32 + lane;            // key row inside the tile
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t myS = tS + lane_off + cg * 32, mydP = tdP + lane_off + cg * 32;
    const float c = p.scale * kLog2e;
    bool ok = true;
    for (int it = 0; it < iters && ok; ++it) {
      const int i = i0 + it % per_head;
      const int st = it & 1;
      const bool diag = p.causal && i == j;
      ok = mbar_wait(&bar->q_full[st], (it >> 1) & 1, &bar->abort_flag, p.status, 140);   // statistics
      if (!ok) break;
      ok = mbar_wait(&bar->s_full, it & 1, &bar->abort_flag, p.status, 141);
      if (!ok) break;
      tc_fence_after();
      float pr[32];
      {
        uint32_t s[32];
        tmem_ld_32x32(myS, s);
        const float4* L4 = reinterpret_cast<const float4*>(stats + st * 2 * BT + cg * 32);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 l = L4[g];
          pr[4 * g] = exp2_mixed<POLY>(fmaf(__uint_as_float(s[4 * g]), c, -l.x), 4 * g);
          pr[4 * g + 1] = exp2_mixed<POLY>(fmaf(__uint_as_float(s[4 * g + 1]), c, -l.y), 4 * g + 1);
          pr[4 * g + 2] = exp2_mixed<POLY>(fmaf(__uint_as_float(s[4 * g + 2]), c, -l.z), 4 * g + 2);
          pr[4 * g + 3] = exp2_mixed<POLY>(fmaf(__uint_as_float(s[4 * g + 3]), c, -l.w), 4 * g + 3);
        }
      }
      if (diag) {
        // query cg * 32 + k sees key `row` only if it is not earlier than the key
#pragma unroll
        for (int k = 0; k < 32; ++k)
          if (cg * 32 + k < row) pr[k] = 0.f;
      }
      {
        uint32_t packed[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) packed[k] = pack_bf16x2(pr[2 * k], pr[2 * k + 1]);
        tmem_st_32x16(myS, packed);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->p_full);
      ok = mbar_wait(&bar->dp_full, it & 1, &bar->abort_flag, p.status, 142);
      if (!ok) break;
      tc_fence_after();
      {
        uint32_t dp[32];
        tmem_ld_32x32(mydP, dp);
        const float4* D4 = reinterpret_cast<const float4*>(stats + st * 2 * BT + BT + cg * 32);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 l = D4[g];
          packed[2 * g] = pack_bf16x2(pr[4 * g] * (__uint_as_float(dp[4 * g]) - l.x),
                                      pr[4 * g + 1] * (__uint_as_float(dp[4 * g + 1]) - l.y));
          packed[2 * g + 1] = pack_bf16x2(pr[4 * g + 2] * (__uint_as_float(dp[4 * g + 2]) - l.z),
                                          pr[4 * g + 3] * (__uint_as_float(dp[4 * g + 3]) - l.w));
        }
        tmem_st_32x16(mydP, packed);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->ds_full);
    }
    if (ok) ok = mbar_wait(&bar->acc_done, 0, &bar->abort_flag, p.status, 143);
    if (ok) {
      tc_fence_after();
      const long long t = kv_row0 + row;
      if (cg * 32 < D) {
        store_cols32(tdV + lane_off + cg * 32, p.dv + t * p.dv_row + (long long)hkv * p.dv_head + cg * 32, 1.f);
        store_cols32(tdK + lane_off + cg * 32, p.dk + t * p.dk_row + (long long)hkv * p.dk_head + cg * 32, p.scale);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------
// dQ kernel: one CTA per (query tile i, head, batch) sweeps the kv tiles j <= i.
// ---------------------------------------------------------------------------
constexpr int K_STAGES = 3, V_STAGES = 2;
struct QSmem {
  static constexpr int TILE_BYTES = (2 + K_STAGES + V_STAGES) * T_BYTES;
  static constexpr int TOTAL = 1024 + TILE_BYTES + 256;
};
struct QBarriers {
  uint64_t qdo_full;
  uint64_t k_full[K_STAGES], k_empty[K_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
  // dp_full / ds_full: one per dP buffer.  A softmax warp may run one iteration ahead of another (S and dP
  // of the next key tile are issued as soon as S of this one is in registers); with a single "dS written"
  // barrier its arrival for the next tile would complete the phase that the slower warp has not arrived
  // for yet (ops/attention_model.py reproduces that).
  uint64_t s_full, p_done, dp_full[2], ds_full[2], acc_done;
  uint32_t tmem_base;
  volatile int abort_flag;
};

template <bool POLY>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_bwd2_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const Bwd2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = tiles;
  uint8_t* sdO = sQ + T_BYTES;
  uint8_t* sK = sdO + T_BYTES;
  uint8_t* sV = sK + K_STAGES * T_BYTES;
  QBarriers* bar = reinterpret_cast<QBarriers*>(tiles + QSmem::TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nT = p.S / BT;
  const int id = blockIdx.x;
  const int hb = id % (p.Hq * p.batch);
  const int i = nT - 1 - id / (p.Hq * p.batch);       // long sweeps first
  const int h = hb % p.Hq, b = hb / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int nblocks = p.causal ? i + 1 : nT;
  const int q_row0 = b * p.S + i * BT;
  const int kv_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(&bar->qdo_full, 1);
    for (int s = 0; s < K_STAGES; ++s) { mbar_init(&bar->k_full[s], 1); mbar_init(&bar->k_empty[s], 1); }
    for (int s = 0; s < V_STAGES; ++s) { mbar_init(&bar->v_full[s], 1); mbar_init(&bar->v_empty[s], 1); }
    mbar_init(&bar->s_full, 1); mbar_init(&bar->p_done, SOFTMAX_WARPS);
    mbar_init(&bar->dp_full[0], 1); mbar_init(&bar->dp_full[1], 1);
    mbar_init(&bar->ds_full[0], SOFTMAX_WARPS); mbar_init(&bar->ds_full[1], SOFTMAX_WARPS);
    mbar_init(&bar->acc_done, 1);
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bar->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;
  const uint32_t tS = tmem_base, tdP0 = tmem_base + 128, tdQ = tmem_base + 384;     // dP: two buffers of 128

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v); tma_prefetch_desc(&tmap_do);
      mbar_expect_tx(&bar->qdo_full, 2 * T_BYTES);
#pragma unroll
      for (int c = 0; c < DCH; ++c) {
        tma_load_3d(sQ + c * (BT * 128), &tmap_q, &bar->qdo_full, c * 64, q_row0, h);
        tma_load_3d(sdO + c * (BT * 128), &tmap_do, &bar->qdo_full, c * 64, q_row0, h);
      }
      bool ok = true;
      for (int jj = 0; jj < nblocks && ok; ++jj) {
        const int ks = jj % K_STAGES, vs = jj % V_STAGES;
        const uint32_t kph = (jj / K_STAGES) & 1, vph = (jj / V_STAGES) & 1;
        ok = mbar_wait(&bar->k_empty[ks], kph ^ 1, &bar->abort_flag, p.status, 151);
        if (!ok) break;
        mbar_expect_tx(&bar->k_full[ks], T_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sK + ks * T_BYTES + c * (BT * 128), &tmap_k, &bar->k_full[ks], c * 64, kv_base + jj * BT, hkv);
        ok = mbar_wait(&bar->v_empty[vs], vph ^ 1, &bar->abort_flag, p.status, 152);
        if (!ok) break;
        mbar_expect_tx(&bar->v_full[vs], T_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sV + vs * T_BYTES + c * (BT * 128), &tmap_v, &bar->v_full[vs], c * 64, kv_base + jj * BT, hkv);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t aQ = smem_u32(sQ), adO = smem_u32(sdO), aK = smem_u32(sK), aV = smem_u32(sV);
      bool ok = mbar_wait(&bar->qdo_full, 0, &bar->abort_flag, p.status, 153);
      // S(jj) and dP(jj) -> dP buffer jj & 1; the caller has waited for what they overwrite
      auto issue_s_dp = [&](int jj) -> bool {
        const int ks = jj % K_STAGES, vs = jj % V_STAGES;
        if (!mbar_wait(&bar->k_full[ks], (jj / K_STAGES) & 1, &bar->abort_flag, p.status, 154)) return false;
        tc_fence_after();
        issue_kmajor(tS, aQ, aK + ks * T_BYTES);
        umma_commit(&bar->s_full);
        if (!mbar_wait(&bar->v_full[vs], (jj / V_STAGES) & 1, &bar->abort_flag, p.status, 155)) return false;
        tc_fence_after();
        issue_kmajor(tdP0 + (jj & 1) * 128, adO, aV + vs * T_BYTES);
        umma_commit(&bar->dp_full[jj & 1]);
        umma_commit(&bar->v_empty[vs]);
        return true;
      };
      if (ok) ok = issue_s_dp(0);
      for (int jj = 0; jj < nblocks && ok; ++jj) {
        ok = mbar_wait(&bar->p_done, jj & 1, &bar->abort_flag, p.status, 156);      // S(jj) is in registers
        if (!ok) break;
        if (jj + 1 < nblocks) {
          ok = issue_s_dp(jj + 1);
          if (!ok) break;
        }
        ok = mbar_wait(&bar->ds_full[jj & 1], (jj >> 1) & 1, &bar->abort_flag, p.status, 157);
        if (!ok) break;
        tc_fence_after();
        issue_from_tmem(tdQ, tdP0 + (jj & 1) * 128, aK + (jj % K_STAGES) * T_BYTES, jj > 0);   // dQ += dS K
        umma_commit(&bar->k_empty[jj % K_STAGES]);
      }
      if (ok) umma_commit(&bar->acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int cg = (warp - 2) >> 2;                 // 32-column group (keys) of this warp
    const int row = quarter * 32 + lane;            // query row inside the tile
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t myS = tS + lane_off + cg * 32;
    const float c = p.scale * kLog2e;
    const size_t stat = ((size_t)b * p.Hq + h) * p.S + i * BT + row;
    const float lse2 = __ldg(p.lse2 + stat);
    const float delta = __ldg(p.delta + stat);
    bool ok = true;
    for (int jj = 0; jj < nblocks && ok; ++jj) {
      const bool diag = p.causal && jj == i;
      ok = mbar_wait(&bar->s_full, jj & 1, &bar->abort_flag, p.status, 158);
      if (!ok) break;
      tc_fence_after();
      float pr[32];
      {
        uint32_t s[32];
        tmem_ld_32x32(myS, s);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar->p_done);
#pragma unroll
        for (int k = 0; k < 32; ++k) pr[k] = exp2_mixed<POLY>(fmaf(__uint_as_float(s[k]), c, -lse2), k);
      }
      if (diag) {
#pragma unroll
        for (int k = 0; k < 32; ++k)
          if (cg * 32 + k > row) pr[k] = 0.f;
      }
      ok = mbar_wait(&bar->dp_full[jj & 1], (jj >> 1) & 1, &bar->abort_flag, p.status, 159);
      if (!ok) break;
      tc_fence_after();
      {
        const uint32_t mydP = tdP0 + (jj & 1) * 128 + lane_off + cg * 32;
        uint32_t dp[32];
        tmem_ld_32x32(mydP, dp);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int k = 0; k < 16; ++k)
          packed[k] = pack_bf16x2(pr[2 * k] * (__uint_as_float(dp[2 * k]) - delta),
                                  pr[2 * k + 1] * (__uint_as_float(dp[2 * k + 1]) - delta));
        tmem_st_32x16(mydP, packed);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->ds_full[jj & 1]);
    }
    if (ok) ok = mbar_wait(&bar->acc_done, 0, &bar->abort_flag, p.status, 160);
    if (ok) {
      tc_fence_after();
      const long long t = q_row0 + row;
      if (cg * 32 < D)
        store_cols32(tdQ + lane_off + cg * 32, p.dq + t * p.dq_row + (long long)h * p.dq_head + cg * 32, p.scale);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// Same contract as dd_attn_bwd; `scratch` holds 2 * batch * Hq * S floats (delta, then the
// log-sum-exp in base 2).
int run(const void* q, long long q_row, long long q_head, const void* k, long long k_row,
                        long long k_head, const void* v, long long v_row, long long v_head, const void* out,
                        const void* dout, const float* lse, float* scratch, void* dq, long long dq_row,
                        long long dq_head, void* dk, long long dk_row, long long dk_head, void* dv, long long dv_row,
                        long long dv_head, int batch, int S, int Hq, int Hkv, int Dh, int causal, float scale,
                        void* stream) {
  if (S % 128 != 0 || Dh != D || Hq % Hkv != 0 || batch <= 0) return DD_ERR_BAD_ARG;
  if ((dq_row | dq_head | dk_row | dk_head | dv_row | dv_head) % 8) return DD_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv) |
       reinterpret_cast<uintptr_t>(scratch)) & 15)
    return DD_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const uint64_t tokens = (uint64_t)batch * S;
  const long long rows = (long long)tokens * Hq;
  float* delta = scratch;
  float* lse2 = scratch + (size_t)batch * Hq * S;
  attn_prepass_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(out),
                                                               reinterpret_cast<const __nv_bfloat16*>(dout), lse, delta,
                                                               lse2, batch, S, Hq);
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
  Bwd2Params p;
  p.lse2 = lse2; p.delta = delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq); p.dq_row = dq_row; p.dq_head = dq_head;
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk); p.dk_row = dk_row; p.dk_head = dk_head;
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv); p.dv_row = dv_row; p.dv_head = dv_head;
  p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.batch = batch; p.causal = causal; p.scale = scale;
  p.status = device_status(&err);
  if (err) return err;
  // DISTDL_ATTN_EXP_POLY=1: a third of the exponentials on the FMA pipe (see exp2_fma)
  static const bool poly = [] { const char* e = getenv("DISTDL_ATTN_EXP_POLY"); return e != nullptr && e[0] == '1'; }();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd2_dkdv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         KVSmem::TOTAL);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_bwd2_dkdv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, KVSmem::TOTAL);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_bwd2_dq_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, QSmem::TOTAL);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_bwd2_dq_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, QSmem::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  const int nT = S / BT;
  if (poly) {
    attn_bwd2_dkdv_kernel<true><<<nT * Hkv * batch, NUM_THREADS, KVSmem::TOTAL, s>>>(tq, tk, tv, tdo, p);
    attn_bwd2_dq_kernel<true><<<nT * Hq * batch, NUM_THREADS, QSmem::TOTAL, s>>>(tq, tk, tv, tdo, p);
  } else {
    attn_bwd2_dkdv_kernel<false><<<nT * Hkv * batch, NUM_THREADS, KVSmem::TOTAL, s>>>(tq, tk, tv, tdo, p);
    attn_bwd2_dq_kernel<false><<<nT * Hq * batch, NUM_THREADS, QSmem::TOTAL, s>>>(tq, tk, tv, tdo, p);
  }
  return (int)cudaGetLastError();
}

}  // namespace DD_BWD2_NS
