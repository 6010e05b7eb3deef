// Definitions shared by the fused compute + collective GEMM kernels
// (single-CTA tiles in gemm_fused.cu, CTA-pair tiles in gemm_fused2.cu).
#pragma once

#include "gemm_tcgen05.cuh"

namespace dd {
namespace fused {

using namespace dd::gemm;

constexpr int kMaxPeers = 8;
constexpr int FUSED_THREADS = NUM_THREADS + 128;   // + 4 comm warps (ag_gemm)
constexpr int kReduceCtas = 592;

// word offsets inside a signal pad (uint32 units); the first 1024 words belong
// to the standalone collectives
constexpr int PAD_AG = 1024;          // [writer]: ag_gemm start / end signals
constexpr int PAD_RS_DELIVERED = 1040;  // [parity * 8 + writer]
constexpr int PAD_RS_CONSUMED = 1072;   // [parity * 8 + writer]

struct Geometry {
  int P, me;            // team size, my index
  int batch;            // batch entries
  int s_local;          // rows per (batch entry, member); multiple of 128
  __device__ __forceinline__ int blocks_per_seg() const { return s_local / BM; }
  __device__ __forceinline__ int row_blocks() const { return batch * P * blocks_per_seg(); }
  // order index -> row-block; `first` is the member whose blocks come first
  __device__ __forceinline__ int block_of(int o, int first, int& owner, int& local_block) const {
    const int q = blocks_per_seg();
    const int per_member = batch * q;
    const int rr = o / per_member, rem = o - rr * per_member;
    const int bi = rem / q, j = rem - bi * q;
    owner = (rr + first) % P;
    local_block = bi * q + j;                    // block index inside the owner's shard
    return bi * (P * q) + owner * q + j;         // block index in the gathered matrix
  }
};

__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void red_release_sys(uint32_t* p) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ void proxy_fence_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Bounded spin until *p (as a counter) has reached `want`.
__host__ __device__ constexpr int wait_slot(int where) {
  return (where == 201 || where == 231) ? 0 : (where == 202 || where == 232) ? 1 : (where == 203 || where == 233) ? 2
         : (where == 241 || where == 211) ? 3 : 4;
}

template <bool SYS>
__device__ __forceinline__ bool wait_counter(const uint32_t* p, uint32_t want, volatile int* abort_flag,
                                             StatusRecord* st, int where) {
  uint32_t seen = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
  if ((int32_t)(seen - want) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    seen = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if ((int32_t)(seen - want) >= 0) {
      if (blockIdx.x == 0) account_wait(st, wait_slot(where), globaltimer_ns() - t0);
      return true;
    }
    if ((++it & 0x3f) == 0) {
      if (*abort_flag) return false;
      // a wait that ran out earlier (in this or a previous kernel) leaves the counters out of
      // step: fail at once instead of spending the full limit again in every later kernel
      if (st != nullptr && *reinterpret_cast<volatile int*>(&st->code) != 0) {
        *abort_flag = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > kSpinLimitNs) {
        *abort_flag = 1;
        report_timeout(st, where, (int)want, (int)seen);
        return false;
      }
    }
  }
}

struct AgParams {
  Params g;                          // GEMM part (M = batch * P * s_local)
  Geometry geo;
  const void* shard[kMaxPeers];      // member i's shard [batch*s_local, K] (peer-mapped; [me] = local)
  __nv_bfloat16* G;                  // gathered activation [M, K], local
  uint32_t* ready;                   // [row_blocks] words, local; value == epoch when the block is in G
  uint32_t epoch;
  uint32_t* pad[kMaxPeers];          // signal pads (peer-mapped)
  int writer[kMaxPeers];             // writer index of member i
  uint32_t expect[kMaxPeers];        // value of member i's "shard is staged" signal for this call
  uint32_t* done_counter;            // local: CTAs that finished pulling (monotone)
  uint32_t done_target;              // value of done_counter when all CTAs of this call are through
  // CTA-pair kernel only: row blocks are pulled in kPullSub pieces by different CTAs;
  // ready_cnt[rb] counts the pieces of this call (the last arrival resets it).
  uint32_t* ready_cnt;
  // Value of member i's pad word that the kernel waits for before it exits: its
  // "done pulling" signal of THIS call (single staging buffer), or of the previous
  // call when the shard staging is double buffered (already there in practice).
  uint32_t end_expect[kMaxPeers];
};
constexpr int kPullSub = 4;          // pieces per 128-row block (32 rows each)


// Output tensor maps of the CTA-pair kernels, box = 64 columns x 32 rows of bf16.
// gemm_rs: m[i] = member i's staging slot for source `me`, [batch*s_local rows][N];
// ag_gemm: m[0] = the output D.
struct RsOutMaps {
  CUtensorMap m[kMaxPeers];
};

struct RsParams {
  Params g;                          // GEMM part; g.D unused
  Geometry geo;
  __nv_bfloat16* slot[kMaxPeers];    // member i's staging, slot [source = me]: [batch*s_local, N] (peer-mapped)
  uint32_t* pad[kMaxPeers];
  int writer[kMaxPeers];
  int parity;
  uint32_t consumed_expect[kMaxPeers];  // peer i must have consumed the previous use of this parity
  uint32_t* done_counter;            // local, monotone
  uint32_t done_target;
  int tma_store;                     // pair kernel: write the tiles with TMA stores from shared memory
  // pair kernel with the fold inside the GEMM: the tiles of this member's own rows add the
  // partials that the peers delivered (my_slot[i] = local staging slot of source i) and go
  // straight to the output (omaps.m[me]); no separate reduction kernel.
  int fold;
  const __nv_bfloat16* my_slot[kMaxPeers];
  uint32_t delivered_expect[kMaxPeers];
  uint32_t* done_counter2;           // local, monotone: CTAs through with their own tiles
  uint32_t done_target2;
};


}  // namespace fused
}  // namespace dd

// CTA-pair launchers (gemm_fused2.cu)
int dd_launch_ag_pair(const CUtensorMap& ta, const CUtensorMap& tb, const dd::fused::RsOutMaps& om,
                      const dd::fused::AgParams& ap, int w_mn, int ctas, cudaStream_t s);
int dd_launch_rs_pair(const CUtensorMap& ta, const CUtensorMap& tb, const dd::fused::RsOutMaps& om,
                      const dd::fused::RsParams& rp, int w_mn, int ctas, cudaStream_t s);
