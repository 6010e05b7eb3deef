// Flash attention forward, two query tiles per CTA ("ping-pong"); head dim DD_HEAD_DIM (128 or 64:
// this file is included once per head dimension by attention_fwd2.cu, inside namespace DD_FWD2_NS).
//
// One CTA handles 256 query rows of one (batch, head) as two 128-row tiles:
//   warp 0        TMA producer: both Q tiles once, then K_j / V_j (2-stage rings)
//   warp 1        MMA issuer:   S_t = Q_t K_j^T and O_t += P_t V_j for t = 0, 1
//   warps 2..5    softmax of tile 0 (one thread per query row)
//   warps 6..9    softmax of tile 1
// Tensor memory (512 columns): S_0 | S_1 | O_0 | O_1, 128 fp32 columns each (O_t uses the first
// DD_HEAD_DIM of its 128).  The
// probabilities never touch shared memory: a softmax thread reads its row of S_t
// into registers, and writes P_t (bf16 pairs) back over the first 64 columns of
// S_t with tcgen05.st; the second product takes its A operand from tensor memory.
// O_t stays in tensor memory for the whole row of blocks; it is rescaled only when
// the running maximum has grown by more than 2^8 since the last rescale (the
// probabilities then exceed 1 by at most that factor, which fp32 sums and bf16
// probabilities absorb), and the final 1 / l scaling happens on the way out.
// While tile 0's softmax runs, the tensor cores work on tile 1, and vice versa.
//
// Issue order per KV block j:  PV_0(j), S_0(j+1), PV_1(j), S_1(j+1); products of
// one thread execute in order, so S_t(j+1) may overwrite P_t(j) right after PV_t(j)
// was issued.  Causal: tile t of query pair qp sees blocks 0 .. 2 qp + t.
// All waits are bounded; a timeout drains and frees tensor memory.
namespace DD_FWD2_NS {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int D = DD_HEAD_DIM;
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 320;
constexpr int Q_BYTES = BQ * D * 2;       // one query tile
constexpr int KV_BYTES = BKV * D * 2;
constexpr int TILE_BYTES = 2 * Q_BYTES + 2 * KV_STAGES * KV_BYTES;
constexpr int SMEM_TOTAL = 1024 + TILE_BYTES + 256;

struct Barriers {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2];      // S_t complete (tensor core -> softmax)
  uint64_t p_full[2];      // P_t written, S_t consumed (softmax -> tensor core), 4 warps arrive
  uint64_t pv_done[2];     // O_t += P_t V complete
  uint32_t tmem_base;
  volatile int abort_flag;
};

struct Params2 {
  __nv_bfloat16* O;     // [tokens][Hq][D]
  float* lse;           // [batch][Hq][S]
  int S, Hq, Hkv, batch;
  int causal;
  float scale;
  StatusRecord* status;
};

template <bool POLY>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const Params2 p) {
  constexpr int DCH = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = tiles;                          // two tiles back to back
  uint8_t* sK = sQ + 2 * Q_BYTES;
  uint8_t* sV = sK + KV_STAGES * KV_BYTES;
  Barriers* bar = reinterpret_cast<Barriers*>(tiles + TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nQP = p.S / (2 * BQ);
  // heaviest query pairs first; heads vary fastest (kv heads shared through L2)
  const int id = blockIdx.x;
  const int hb = id % (p.Hq * p.batch);
  const int qp = nQP - 1 - id / (p.Hq * p.batch);
  const int h = hb % p.Hq, b = hb / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int nkv = p.S / BKV;
  const int n0 = p.causal ? 2 * qp + 1 : nkv;      // blocks seen by tile 0
  const int n1 = p.causal ? 2 * qp + 2 : nkv;      // blocks seen by tile 1 (>= n0)
  const int q_row0 = b * p.S + qp * 2 * BQ;
  const int kv_row0 = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bar->k_full[s], 1); mbar_init(&bar->k_empty[s], 1);
      mbar_init(&bar->v_full[s], 1); mbar_init(&bar->v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&bar->s_full[t], 1);
      mbar_init(&bar->p_full[t], 4);
      mbar_init(&bar->pv_done[t], 1);
    }
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bar->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
      mbar_expect_tx(&bar->q_full, 2 * Q_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sQ + t * Q_BYTES + c * (BQ * 128), &tmap_q, &bar->q_full, c * 64, q_row0 + t * BQ, h);
      bool ok = true;
      for (int j = 0; j < n1 && ok; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        ok = mbar_wait(&bar->k_empty[st], ph ^ 1, &bar->abort_flag, p.status, 31);
        if (!ok) break;
        mbar_expect_tx(&bar->k_full[st], KV_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sK + st * KV_BYTES + c * (BKV * 128), &tmap_k, &bar->k_full[st], c * 64, kv_row0 + j * BKV, hkv);
        ok = mbar_wait(&bar->v_empty[st], ph ^ 1, &bar->abort_flag, p.status, 32);
        if (!ok) break;
        mbar_expect_tx(&bar->v_full[st], KV_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sV + st * KV_BYTES + c * (BKV * 128), &tmap_v, &bar->v_full[st], c * 64, kv_row0 + j * BKV, hkv);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);   // Q, K both K-major
      constexpr uint32_t idesc_pv = make_idesc_bf16(BQ, D, 0, 1);    // P (tensor memory), V MN-major
      bool ok = mbar_wait(&bar->q_full, 0, &bar->abort_flag, p.status, 33);
      // S_t(j) = Q_t K_j^T; the caller has made sure that K_j is in shared memory
      auto issue_S = [&](int t, int j) {
        const int st = j % KV_STAGES;
        const uint32_t q_addr = smem_u32(sQ + t * Q_BYTES), k_addr = smem_u32(sK + st * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
          umma_f16(tmem_base + t * 128, make_smem_desc_sw128(q_addr + off, 16, 1024),
                   make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bar->s_full[t]);
      };
      auto issue_PV = [&](int t, int j) {
        const int st = j % KV_STAGES;
        const uint32_t v_addr = smem_u32(sV + st * KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk)      // 16 kv rows = 8 columns of packed P
          umma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + kk * 8,
                      make_smem_desc_sw128(v_addr + kk * (16 * 128), BKV * 128, 1024), idesc_pv,
                      (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&bar->pv_done[t]);
      };
      if (ok) ok = mbar_wait(&bar->k_full[0], 0, &bar->abort_flag, p.status, 34);
      if (ok) {
        tc_fence_after();
        issue_S(0, 0);
        issue_S(1, 0);
      }
      for (int j = 0; j < n1 && ok; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const int stn = (j + 1) % KV_STAGES;
        const uint32_t phn = ((j + 1) / KV_STAGES) & 1;
        ok = mbar_wait(&bar->v_full[st], ph, &bar->abort_flag, p.status, 35);
        if (!ok) break;
        bool k_next_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          const int nt = t == 0 ? n0 : n1;
          if (j >= nt) continue;
          ok = mbar_wait(&bar->p_full[t], j & 1, &bar->abort_flag, p.status, 36);
          if (!ok) break;
          tc_fence_after();
          issue_PV(t, j);
          if (j + 1 < nt) {
            if (!k_next_ready) {
              ok = mbar_wait(&bar->k_full[stn], phn, &bar->abort_flag, p.status, 37);
              if (!ok) break;
              tc_fence_after();
              k_next_ready = true;
            }
            issue_S(t, j + 1);
          }
        }
        if (!ok) break;
        // V_j is free once the products of both tiles are through; K_j was last read by
        // the S products of block j, which precede these commits in issue order
        umma_commit(&bar->v_empty[st]);
        umma_commit(&bar->k_empty[st]);
      }
    }
  } else {
    // -------------------------------- softmax --------------------------------
    const int t = (warp - 2) >> 2;                  // query tile of this warpgroup
    const int quarter = warp & 3;                   // tensor-memory lane quarter this warp may access
    const int row = quarter * 32 + lane;            // row inside the tile
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem_base + t * 128 + lane_off;
    const uint32_t tO = tmem_base + 256 + t * 128 + lane_off;
    const int nt = t == 0 ? n0 : n1;
    const int diag = p.causal ? 2 * qp + t : -1;
    const float c = p.scale * 1.4426950408889634f;  // scores are exponentiated base 2
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nt && ok; ++j) {
      ok = mbar_wait(&bar->s_full[t], j & 1, &bar->abort_flag, p.status, 38);
      if (!ok) break;
      tc_fence_after();
      uint32_t s[128];
      tmem_ld_32x32(tS, *reinterpret_cast<uint32_t(*)[32]>(s));
      tmem_ld_32x32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(s + 32));
      tmem_ld_32x32(tS + 64, *reinterpret_cast<uint32_t(*)[32]>(s + 64));
      tmem_ld_32x32(tS + 96, *reinterpret_cast<uint32_t(*)[32]>(s + 96));
      tmem_ld_wait();
      float mx = m_ref;
      if (j == diag) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          if (i > row) s[i] = 0xff800000u;          // -inf
          mx = fmaxf(mx, __uint_as_float(s[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i) mx = fmaxf(mx, __uint_as_float(s[i]));
      }
      // rescale O only when the maximum moved by more than 2^8 (whole warp together:
      // the tensor-memory accesses are warp-wide)
      const bool grow = (j > 0) && ((mx - m_ref) * c > 8.f);
      if (j == 0) m_ref = mx;
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? exp2f((m_ref - mx) * c) : 1.f;
        if (grow) { m_ref = mx; l *= alpha; }
        ok = mbar_wait(&bar->pv_done[t], (j - 1) & 1, &bar->abort_flag, p.status, 39);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t r[32];
          tmem_ld_32x32(tO + ch * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32(tO + ch * 32, r);
        }
        tmem_st_wait();
      }
      const float mc = m_ref * c;
      float lsum = 0.f;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = exp2_mixed<POLY>(__uint_as_float(s[ch * 32 + i]) * c - mc, i);
          const float p1 = exp2_mixed<POLY>(__uint_as_float(s[ch * 32 + i + 1]) * c - mc, i + 1);
          lsum += p0 + p1;
          packed[i >> 1] = pack_bf16x2(p0, p1);
        }
        tmem_st_32x16(tS + ch * 16, packed);
      }
      l += lsum;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->p_full[t]);
    }
    if (ok) {
      ok = mbar_wait(&bar->pv_done[t], (nt - 1) & 1, &bar->abort_flag, p.status, 40);
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / l;
        __nv_bfloat16* orow = p.O + ((size_t)(q_row0 + t * BQ + row) * p.Hq + h) * D;
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t r[32];
          tmem_ld_32x32(tO + ch * 32, r);
          tmem_ld_wait();
          uint4* dst = reinterpret_cast<uint4*>(orow + ch * 32);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * g]) * inv, __uint_as_float(r[8 * g + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * inv, __uint_as_float(r[8 * g + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * inv, __uint_as_float(r[8 * g + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * inv, __uint_as_float(r[8 * g + 7]) * inv);
            dst[g] = v;
          }
        }
        if (p.lse != nullptr)
          p.lse[((size_t)b * p.Hq + h) * p.S + qp * 2 * BQ + t * BQ + row] = m_ref * p.scale + logf(l);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// Two-tile forward kernel: sequence length a multiple of 256.  Same argument convention as dd_attn_fwd.
int run(const void* q, long long q_row_stride, long long q_head_stride, const void* k,
                        long long k_row_stride, long long k_head_stride, const void* v, long long v_row_stride,
                        long long v_head_stride, void* out, float* lse, int batch, int S, int Hq, int Hkv, int Dh,
                        int causal, float scale, void* stream) {
  if (S % 256 != 0 || Dh != D || Hq % Hkv != 0 || batch <= 0) return DD_ERR_BAD_ARG;
  const uint64_t tokens = (uint64_t)batch * S;
  CUtensorMap tq, tk, tv;
  int r = get_tensor_map_bf16_3d(&tq, q, D, tokens, Hq, q_row_stride * 2, q_head_stride * 2, 64, BQ);
  if (r) return r;
  r = get_tensor_map_bf16_3d(&tk, k, D, tokens, Hkv, k_row_stride * 2, k_head_stride * 2, 64, BKV);
  if (r) return r;
  r = get_tensor_map_bf16_3d(&tv, v, D, tokens, Hkv, v_row_stride * 2, v_head_stride * 2, 64, BKV);
  if (r) return r;
  int err = 0;
  Params2 p;
  p.O = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.batch = batch; p.causal = causal; p.scale = scale;
  p.status = device_status(&err);
  if (err) return err;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  // DISTDL_ATTN_EXP_POLY=1: a third of the exponentials on the FMA pipe (exp2_fma in common.cuh)
  static const bool poly = [] { const char* e = getenv("DISTDL_ATTN_EXP_POLY"); return e != nullptr && e[0] == '1'; }();
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_fwd2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  const int grid = (S / (2 * BQ)) * Hq * batch;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (poly) attn_fwd2_kernel<true><<<grid, NUM_THREADS, SMEM_TOTAL, st>>>(tq, tk, tv, p);
  else attn_fwd2_kernel<false><<<grid, NUM_THREADS, SMEM_TOTAL, st>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

}  // namespace DD_FWD2_NS
