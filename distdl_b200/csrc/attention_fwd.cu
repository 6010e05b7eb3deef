// Causal / full flash attention forward for sm_100a on tcgen05 + TMEM + TMA.
//
// One CTA handles one 128-row query tile of one (batch, head):
//   warp 0      TMA producer: Q once, then K_j and V_j tiles (2-stage rings)
//   warp 1      MMA issuer:   S_j = Q K_j^T  (TMEM, double buffered)
//                             R_j = P_j V_j  (TMEM, fresh accumulator per block)
//   warps 2..5  softmax: each thread owns one query row: reads its S row from
//               TMEM, keeps the running max / sum, writes P_j (bf16) into
//               shared memory in the 128B-swizzled layout the tensor core
//               expects, and accumulates O = O * alpha + R_j in registers.
// The issue order S_0, S_1, PV_0, S_2, PV_1, ... lets the next score tile run on
// the tensor cores while the softmax warps work on the current one.
//
// q, k, v are addressed as [token][head][D] with arbitrary token/head strides
// (so a packed qkv projection output is consumed in place); grouped-query
// attention maps query head h to kv head h / (Hq / Hkv).  Sequence length must
// be a multiple of 128.  Output: O [token][Hq][D] bf16 and the row-wise
// log-sum-exp (natural log, of the scaled scores) for the backward pass.
#include "common.cuh"
#include "runtime.cuh"

using namespace dd;

namespace {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 192;

template <int D>
struct FwdSmem {
  static constexpr int Q_BYTES = BQ * D * 2;
  static constexpr int KV_BYTES = BKV * D * 2;
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int TILE_BYTES = Q_BYTES + 2 * KV_STAGES * KV_BYTES + P_BYTES;
  static constexpr int TOTAL = 1024 + TILE_BYTES + 256;
};

struct FwdBarriers {
  uint64_t q_full;
  uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
  uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full;
  uint64_t pv_done;
  uint32_t tmem_base;
  volatile int abort_flag;
};

struct FwdParams {
  __nv_bfloat16* O;     // [tokens][Hq][D]
  float* lse;           // [batch][Hq][S]
  int S, Hq, Hkv, batch;
  int causal;
  float scale;          // softmax scale
  StatusRecord* status;
};

template <int D>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  using SM = FwdSmem<D>;
  constexpr int DCH = D / 64;  // 64-element (128 B) chunks along the head dimension
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = tiles;
  uint8_t* sK = sQ + SM::Q_BYTES;
  uint8_t* sV = sK + KV_STAGES * SM::KV_BYTES;
  uint8_t* sP = sV + KV_STAGES * SM::KV_BYTES;
  FwdBarriers* bar = reinterpret_cast<FwdBarriers*>(tiles + SM::TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nQ = p.S / BQ;
  // heaviest query tiles first; heads vary fastest so that the query heads of
  // one kv group run together and share K/V in L2
  const int id = blockIdx.x;
  const int hb = id % (p.Hq * p.batch);
  const int qb = nQ - 1 - id / (p.Hq * p.batch);
  const int h = hb % p.Hq, b = hb / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int nblocks = p.causal ? qb + 1 : p.S / BKV;
  const int q_row0 = b * p.S + qb * BQ;
  const int kv_row0 = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(&bar->q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&bar->k_full[s], 1); mbar_init(&bar->k_empty[s], 1);
      mbar_init(&bar->v_full[s], 1); mbar_init(&bar->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(&bar->s_full[s], 1); mbar_init(&bar->s_empty[s], 4); }
    mbar_init(&bar->p_full, 4);
    mbar_init(&bar->pv_done, 1);
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bar->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;
  const uint32_t tmem_S = tmem_base;            // 2 x 128 columns
  const uint32_t tmem_R = tmem_base + 256;      // D columns

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v);
      mbar_expect_tx(&bar->q_full, SM::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DCH; ++c) tma_load_3d(sQ + c * (BQ * 128), &tmap_q, &bar->q_full, c * 64, q_row0, h);
      bool ok = true;
      for (int j = 0; j < nblocks && ok; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        ok = mbar_wait(&bar->k_empty[st], ph ^ 1, &bar->abort_flag, p.status, 11);
        if (!ok) break;
        mbar_expect_tx(&bar->k_full[st], SM::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sK + st * SM::KV_BYTES + c * (BKV * 128), &tmap_k, &bar->k_full[st], c * 64,
                      kv_row0 + j * BKV, hkv);
        ok = mbar_wait(&bar->v_empty[st], ph ^ 1, &bar->abort_flag, p.status, 12);
        if (!ok) break;
        mbar_expect_tx(&bar->v_full[st], SM::KV_BYTES);
#pragma unroll
        for (int c = 0; c < DCH; ++c)
          tma_load_3d(sV + st * SM::KV_BYTES + c * (BKV * 128), &tmap_v, &bar->v_full[st], c * 64,
                      kv_row0 + j * BKV, hkv);
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BQ, BKV, 0, 0);   // Q, K both K-major
      constexpr uint32_t idesc_pv = make_idesc_bf16(BQ, D, 0, 1);    // P K-major, V MN-major
      bool ok = mbar_wait(&bar->q_full, 0, &bar->abort_flag, p.status, 13);
      auto issue_S = [&](int j) -> bool {
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        const int sb = j & 1;
        if (!mbar_wait(&bar->s_empty[sb], ((j >> 1) & 1) ^ 1, &bar->abort_flag, p.status, 14)) return false;
        if (!mbar_wait(&bar->k_full[st], ph, &bar->abort_flag, p.status, 15)) return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK + st * SM::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
          umma_f16(tmem_S + sb * 128, make_smem_desc_sw128(q_addr + off, 16, 1024),
                   make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bar->k_empty[st]);
        umma_commit(&bar->s_full[sb]);
        return true;
      };
      if (ok) ok = issue_S(0);
      for (int j = 0; j < nblocks && ok; ++j) {
        if (j + 1 < nblocks) { ok = issue_S(j + 1); if (!ok) break; }
        const int st = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        ok = mbar_wait(&bar->v_full[st], ph, &bar->abort_flag, p.status, 16);
        if (!ok) break;
        ok = mbar_wait(&bar->p_full, j & 1, &bar->abort_flag, p.status, 17);
        if (!ok) break;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP), v_addr = smem_u32(sV + st * SM::KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint32_t poff = (kk / 4) * (BQ * 128) + (kk % 4) * 32;   // K-major A
          const uint32_t voff = kk * (16 * 128);                          // MN-major B: 16 kv rows
          umma_f16(tmem_R, make_smem_desc_sw128(p_addr + poff, 16, 1024),
                   make_smem_desc_sw128(v_addr + voff, BKV * 128, 1024), idesc_pv, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bar->v_empty[st]);
        umma_commit(&bar->pv_done);
      }
    }
  } else {
    // ------------------------------- softmax --------------------------------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;            // row inside the query tile
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const float c = p.scale * 1.4426950408889634f;  // scores are exponentiated base 2
    float m = -INFINITY, l = 0.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < nblocks && ok; ++j) {
      const int sb = j & 1;
      ok = mbar_wait(&bar->s_full[sb], (j >> 1) & 1, &bar->abort_flag, p.status, 18);
      if (!ok) break;
      tc_fence_after();
      const bool diag = p.causal && (j == qb);
      const uint32_t taddr = tmem_S + sb * 128 + lane_off;
      // pass 1: row maximum
      float mx = m;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + ch * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float s = __uint_as_float(r[i]);
          if (!diag || (ch * 32 + i) <= row) mx = fmaxf(mx, s);
        }
      }
      const float alpha = exp2f((m - mx) * c);   // m = -inf on the first block gives 0
      m = mx;
      const float mc = mx * c;
      float lsum = 0.f;
      // P buffer is free once the previous PV product has been consumed
      if (j > 0) {
        ok = mbar_wait(&bar->pv_done, (j - 1) & 1, &bar->abort_flag, p.status, 19);
        if (!ok) break;
        tc_fence_after();
        // fold the previous block's PV product into the running output
        // (alpha_prev was applied when that block's P was formed; see below)
      }
      // pass 2: probabilities -> bf16 -> swizzled shared memory
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + ch * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(__uint_as_float(r[i]) * c - mc);
          float p1 = exp2f(__uint_as_float(r[i + 1]) * c - mc);
          if (diag) {
            if (ch * 32 + i > row) p0 = 0.f;
            if (ch * 32 + i + 1 > row) p1 = 0.f;
          }
          lsum += p0 + p1;
          packed[i >> 1] = pack_bf16x2(p0, p1);
        }
        // 32 kv columns = 4 groups of 16 B inside 64-column chunk (ch / 2)
        uint8_t* base = sP + (ch >> 1) * (BQ * 128) + row * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int grp = (ch & 1) * 4 + g;
          uint4 val = make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
          *reinterpret_cast<uint4*>(base + ((grp ^ (row & 7)) << 4)) = val;
        }
      }
      // S buffer may be overwritten by the next-but-one score tile
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->s_empty[sb]);
      // the previous block's PV product (already complete: waited above)
      if (j > 0) {
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_R + lane_off + ch * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[ch * 32 + i] += __uint_as_float(r[i]);
        }
        tc_fence_before();
      }
      // rescale the running output and sum to the new maximum
#pragma unroll
      for (int i = 0; i < D; ++i) o[i] *= alpha;
      l = l * alpha + lsum;
      // publish P: generic-proxy writes must be visible to the tensor core
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->p_full);
    }
    if (ok) {
      ok = mbar_wait(&bar->pv_done, (nblocks - 1) & 1, &bar->abort_flag, p.status, 20);
      if (ok) {
        tc_fence_after();
        const float inv = 1.f / l;
        __nv_bfloat16* orow = p.O + ((size_t)(q_row0 + row) * p.Hq + h) * D;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_R + lane_off + ch * 32, r);
          tmem_ld_wait();
          uint4* dst = reinterpret_cast<uint4*>(orow + ch * 32);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 v;
            v.x = pack_bf16x2((o[ch * 32 + 8 * g] + __uint_as_float(r[8 * g])) * inv,
                              (o[ch * 32 + 8 * g + 1] + __uint_as_float(r[8 * g + 1])) * inv);
            v.y = pack_bf16x2((o[ch * 32 + 8 * g + 2] + __uint_as_float(r[8 * g + 2])) * inv,
                              (o[ch * 32 + 8 * g + 3] + __uint_as_float(r[8 * g + 3])) * inv);
            v.z = pack_bf16x2((o[ch * 32 + 8 * g + 4] + __uint_as_float(r[8 * g + 4])) * inv,
                              (o[ch * 32 + 8 * g + 5] + __uint_as_float(r[8 * g + 5])) * inv);
            v.w = pack_bf16x2((o[ch * 32 + 8 * g + 6] + __uint_as_float(r[8 * g + 6])) * inv,
                              (o[ch * 32 + 8 * g + 7] + __uint_as_float(r[8 * g + 7])) * inv);
            dst[g] = v;
          }
        }
        if (p.lse != nullptr)
          p.lse[((size_t)b * p.Hq + h) * p.S + qb * BQ + row] = m * p.scale + logf(l);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int D>
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
               cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = attn_fwd_kernel<D>;
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<D>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured[dev & 63] = true;
  }
  const int grid = (p.S / BQ) * p.Hq * p.batch;
  kern<<<grid, NUM_THREADS, FwdSmem<D>::TOTAL, stream>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

}  // namespace

// q/k/v: bf16, element (token t, head h, d) at base + t*row_stride + h*head_stride + d
// (strides in elements, multiples of 8; base 16-byte aligned).
DD_API int dd_attn_fwd(const void* q, long long q_row_stride, long long q_head_stride, const void* k,
                       long long k_row_stride, long long k_head_stride, const void* v, long long v_row_stride,
                       long long v_head_stride, void* out, float* lse, int batch, int S, int Hq, int Hkv, int D,
                       int causal, float scale, void* stream) {
  if (S % 128 != 0 || (D != 64 && D != 128) || Hq % Hkv != 0 || batch <= 0) return DD_ERR_BAD_ARG;
  const uint64_t tokens = (uint64_t)batch * S;
  CUtensorMap tq, tk, tv;
  int r = get_tensor_map_bf16_3d(&tq, q, D, tokens, Hq, q_row_stride * 2, q_head_stride * 2, 64, BQ);
  if (r) return r;
  r = get_tensor_map_bf16_3d(&tk, k, D, tokens, Hkv, k_row_stride * 2, k_head_stride * 2, 64, BKV);
  if (r) return r;
  r = get_tensor_map_bf16_3d(&tv, v, D, tokens, Hkv, v_row_stride * 2, v_head_stride * 2, 64, BKV);
  if (r) return r;
  int err = 0;
  FwdParams p;
  p.O = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.batch = batch; p.causal = causal; p.scale = scale;
  p.status = device_status(&err);
  if (err) return err;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  return D == 128 ? launch_fwd<128>(tq, tk, tv, p, s) : launch_fwd<64>(tq, tk, tv, p, s);
}
