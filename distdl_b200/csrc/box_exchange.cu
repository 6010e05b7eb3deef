// Box exchange: strided sub-boxes of local tensors travel between GPUs in ONE
// kernel launch -- pack, peer store, flag, wait, unpack (copy or add), with
// several ordered phases per launch.  It is the data plane of HaloExchange (one
// phase per tensor dimension, so that corners propagate; the adjoint adds the
// ghost regions into the neighbours' bulk and clears them) and of Repartition
// (one phase, every overlap rectangle goes straight from the source tensor to
// the destination tensor).  The reference packs with cupy slicing into send
// buffers, runs grouped ncclSend / ncclRecv, synchronises the host on an event
// and unpacks with slicing again
// (src/distdl/backends/nccl_cupy/functional/halo_exchange.py:49-80,
//  src/distdl/backends/nccl_cupy/functional/repartition.py:142-205).
//
// Protocol.  Every ordered pair (a -> b) of GPUs owns a slot in b's inbox
// region, cut into kBoxBufs chunk buffers.  The chunks that a ever sends to b
// are numbered 0, 1, 2, ... over the life of the process; chunk q uses buffer
// q % kBoxBufs, as its (q / kBoxBufs)-th use.
//   sender:   wait consumed[buf][b] >= use   (b has unpacked the previous use)
//             pack the chunk from the strided box into b's buffer (peer stores)
//             fence, delivered[buf][a] += 1 on b's signal pad
//   receiver: wait delivered[buf][a] >= use + 1
//             unpack the chunk from the local buffer into the strided box
//             consumed[buf][b] += 1 on a's signal pad
// Counters only grow, so nothing is ever reset and a pair needs no barrier;
// members of a team that have nothing to exchange with each other never wait
// for each other.  A chunk is cut into pieces that different CTAs move; the CTA
// that finishes the last piece of a chunk signals.  Half of the CTAs send, the
// other half receive, so a GPU always makes progress on both.  Phases: a work
// item of phase p + 1 starts only after ALL items of phase p of this GPU are
// done (a local counter), because it may read what phase p wrote.
// Every wait is bounded (2 s); on expiry the kernel records where it gave up
// in the status record and all CTAs fall through to the end.
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "runtime.cuh"

using namespace dd;

namespace {

constexpr int kMaxPeers = 8;
constexpr int kBoxBufs = 4;
constexpr int kBoxMaxItems = 48;
constexpr int kBoxCtas = 128;           // half send, half receive
constexpr int kBoxThreads = 256;
// bytes that one CTA moves between two looks at the flags: larger where 16-byte units stream,
// smaller where single elements are gathered (more CTAs share a face)
__host__ __device__ constexpr unsigned long long piece_bytes_for(int unit) { return unit == 16 ? 128 * 1024 : 16 * 1024; }
// word offsets inside a signal pad (uint32 units); [0, 1104) belong to the collectives and the fused GEMMs
constexpr int PAD_BOX_DELIVERED = 1104;   // [buf * 8 + writer]
constexpr int PAD_BOX_CONSUMED = 1136;    // [buf * 8 + writer]

enum { kSend = 0, kRecv = 1, kLocal = 2 };
enum { kAddNone = 0, kAddF32 = 1, kAddBF16 = 2, kAddF16 = 3, kAddF64 = 4 };

// A box of `unit`-byte units inside a tensor: n[3] units along the innermost (contiguous)
// direction, n[0..2] steps along three outer directions with byte strides s[0..2].
struct Box {
  char* base;
  long long s[3];
  int n[4];
  char* lo;                    // the tensor's storage [lo, hi): checked by the bounds-checking build
  char* hi;
};

struct BoxItem {
  Box a;                       // send: source box; recv: destination box; local: source box
  Box b;                       // local copy only: destination box
  unsigned long long bytes;    // message size
  unsigned first_seq;          // number of the first chunk on the ordered pair
  int unit;                    // 16, or the element size
  int unit_b;                  // local copy: unit of the destination side
  int kind, peer, phase;
  int clear_source;            // send: write zeros over the source after reading it
  int add;                     // recv: add into the destination (kAdd*), else overwrite
};

struct BoxArgs {
  BoxItem item[kBoxMaxItems];
  int n_items;
  int n_phases;
  unsigned phase_target[8];    // value of the local progress counter once phase p is complete
  unsigned* progress;          // local, monotone: pieces completed
  unsigned* piece_count;       // local scratch [2][kMaxPeers][kBoxBufs]: pieces of the chunk in flight
  char* inbox[kMaxPeers];      // inbox region of world rank r (peer-mapped); [me] = local
  uint32_t* pad[kMaxPeers];    // signal pads by world rank
  int me;                      // my world rank
  unsigned long long slot_bytes, chunk_bytes;
  StatusRecord* status;
};

__host__ __device__ __forceinline__ char* unit_addr(const Box& x, int unit, unsigned long long g) {
  const unsigned long long n3 = (unsigned long long)x.n[3];
  const unsigned long long i3 = g % n3;
  unsigned long long t = g / n3;
  const unsigned long long i2 = t % (unsigned long long)x.n[2];
  t /= (unsigned long long)x.n[2];
  const unsigned long long i1 = t % (unsigned long long)x.n[1];
  const unsigned long long i0 = t / (unsigned long long)x.n[1];
  return x.base + (long long)i0 * x.s[0] + (long long)i1 * x.s[1] + (long long)i2 * x.s[2] + (long long)i3 * unit;
}

// dst unit (+)= src unit for `unit` in {1, 2, 4, 8, 16}; `zero_src` clears the source afterwards.
__host__ __device__ __forceinline__ void move_unit(char* dst, char* src, int unit, int add, bool zero_src) {
  if (unit == 16) {
    uint4 v = *reinterpret_cast<const uint4*>(src);
    if (add == kAddF32) {
      float4 d = *reinterpret_cast<const float4*>(dst);
      const float4 s = *reinterpret_cast<const float4*>(&v);
      d.x += s.x; d.y += s.y; d.z += s.z; d.w += s.w;
      *reinterpret_cast<float4*>(dst) = d;
    } else if (add == kAddF64) {
      double2 d = *reinterpret_cast<const double2*>(dst);
      const double2 s = *reinterpret_cast<const double2*>(&v);
      d.x += s.x; d.y += s.y;
      *reinterpret_cast<double2*>(dst) = d;
    } else if (add == kAddBF16 || add == kAddF16) {
#ifdef __CUDA_ARCH__
      uint4 d = *reinterpret_cast<const uint4*>(dst);
      uint32_t* dw = reinterpret_cast<uint32_t*>(&d);
      const uint32_t* sw = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (add == kAddBF16) {
          const float2 x = unpack_bf16x2(dw[j]), y = unpack_bf16x2(sw[j]);
          dw[j] = pack_bf16x2(x.x + y.x, x.y + y.y);
        } else {
          const __half2 x = *reinterpret_cast<const __half2*>(&dw[j]), y = *reinterpret_cast<const __half2*>(&sw[j]);
          const float2 fx = __half22float2(x), fy = __half22float2(y);
          const __half2 r = __floats2half2_rn(fx.x + fy.x, fx.y + fy.y);
          dw[j] = *reinterpret_cast<const uint32_t*>(&r);
        }
      }
      *reinterpret_cast<uint4*>(dst) = d;
#endif
    } else {
      *reinterpret_cast<uint4*>(dst) = v;
    }
    if (zero_src) *reinterpret_cast<uint4*>(src) = make_uint4(0, 0, 0, 0);
    return;
  }
  if (add == kAddF32 && unit == 4) {
    *reinterpret_cast<float*>(dst) += *reinterpret_cast<const float*>(src);
  } else if (add == kAddF64 && unit == 8) {
    *reinterpret_cast<double*>(dst) += *reinterpret_cast<const double*>(src);
  } else if ((add == kAddBF16 || add == kAddF16) && unit == 2) {
#ifdef __CUDA_ARCH__
    if (add == kAddBF16) {
      const float r = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(dst)) +
                      __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src));
      *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16(r);
    } else {
      const float r = __half2float(*reinterpret_cast<const __half*>(dst)) +
                      __half2float(*reinterpret_cast<const __half*>(src));
      *reinterpret_cast<__half*>(dst) = __float2half(r);
    }
#endif
  } else {
    switch (unit) {
      case 1: *dst = *src; break;
      case 2: *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<const uint16_t*>(src); break;
      case 4: *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src); break;
      default: *reinterpret_cast<uint64_t*>(dst) = *reinterpret_cast<const uint64_t*>(src); break;
    }
  }
  if (zero_src) {
    switch (unit) {
      case 1: *src = 0; break;
      case 2: *reinterpret_cast<uint16_t*>(src) = 0; break;
      case 4: *reinterpret_cast<uint32_t*>(src) = 0; break;
      default: *reinterpret_cast<uint64_t*>(src) = 0; break;
    }
  }
}

// Bounds-checking build (-DDD_BOUNDS_CHECK, `python -m distdl_b200._build --debug`): an address
// outside the tensor's storage is recorded in the status record (code 1006, the offending unit
// index) and the access is skipped, instead of faulting the GPU.
__device__ __forceinline__ bool in_bounds(const Box& x, const char* p, int unit, StatusRecord* st,
                                          unsigned long long g) {
#ifdef DD_BOUNDS_CHECK
  if (x.lo != nullptr && (p < x.lo || p + unit > x.hi)) {
    if (st != nullptr && atomicCAS(&st->code, 0, DD_ERR_BOUNDS) == 0) {
      st->where = 320;
      st->expected = (int)(g & 0x7fffffff);
      st->seen = (int)(g >> 31);
      __threadfence_system();
    }
    return false;
  }
#endif
  return true;
}

__device__ __forceinline__ void red_release_sys_u32(uint32_t* p) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// 16 bytes from a buffer that another GPU wrote: read at L2, never from a stale L1 line
__device__ __forceinline__ uint4 ld_cg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// Address of row r (all outer indices folded into one number) of a box.
__device__ __forceinline__ char* row_addr(const Box& x, unsigned long long r) {
  if (r <= 0xffffffffull) {             // 32-bit divisions are several times cheaper
    const unsigned r32 = (unsigned)r, n2 = (unsigned)x.n[2], n1 = (unsigned)x.n[1];
    const unsigned i2 = r32 % n2, t = r32 / n2;
    const unsigned i1 = t % n1, i0 = t / n1;
    return x.base + (long long)i0 * x.s[0] + (long long)i1 * x.s[1] + (long long)i2 * x.s[2];
  }
  const unsigned long long i2 = r % (unsigned long long)x.n[2];
  const unsigned long long t = r / (unsigned long long)x.n[2];
  const unsigned long long i1 = t % (unsigned long long)x.n[1];
  const unsigned long long i0 = t / (unsigned long long)x.n[1];
  return x.base + (long long)i0 * x.s[0] + (long long)i1 * x.s[1] + (long long)i2 * x.s[2];
}

// A thread's walk through the units g, g + T, g + 2T, ... of a box (T = threads of the CTA): the row
// and the position inside the row are carried along, so that the divisions of the index arithmetic
// are paid once per thread (and once more only where a step crosses rows of fewer than T units).
struct Cursor {
  unsigned long long row;
  unsigned col;
  char* rowp;
};
__device__ __forceinline__ Cursor cursor_at(const Box& x, unsigned long long g) {
  Cursor c;
  const unsigned n3 = (unsigned)x.n[3];
  c.row = g / n3;
  c.col = (unsigned)(g - c.row * n3);
  c.rowp = row_addr(x, c.row);
  return c;
}
__device__ __forceinline__ void cursor_step(const Box& x, Cursor& c, unsigned step) {
  const unsigned n3 = (unsigned)x.n[3];
  c.col += step;
  if (c.col >= n3) {
    const unsigned adv = c.col / n3;
    c.row += adv;
    c.col -= adv * n3;
    c.rowp = row_addr(x, c.row);
  }
}

// body(box address, unit index g) for every unit g in [lo_u, hi_u) of the box, the threads of the CTA
// sharing the work: consecutive threads take consecutive units (contiguous inside a row).
template <typename Body>
__device__ __forceinline__ void walk_units(const Box& x, int unit, unsigned long long lo_u, unsigned long long hi_u,
                                           Body body) {
  unsigned long long g = lo_u + threadIdx.x;
  if (g >= hi_u) return;
  Cursor c = cursor_at(x, g);
  for (; g < hi_u; g += kBoxThreads) {
    body(c.rowp + (size_t)c.col * unit, g);
    cursor_step(x, c, kBoxThreads);
  }
}

// Plain copy in 16-byte units between a box and a contiguous buffer (`lin` = address of unit 0),
// four vectors per thread in flight.  TO_BOX: the contiguous side is an inbox that another GPU
// wrote (read at L2).
template <bool TO_BOX>
__device__ __forceinline__ void copy16_rows(const Box& x, char* lin, unsigned long long lo_u,
                                            unsigned long long hi_u) {
  unsigned long long g = lo_u + threadIdx.x;
  if (g >= hi_u) return;
  Cursor c = cursor_at(x, g);
  for (; g < hi_u; g += 4ull * kBoxThreads) {
    uint4 v[4];
    char* addr[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const unsigned long long gq = g + (unsigned long long)q * kBoxThreads;
      addr[q] = c.rowp + ((size_t)c.col << 4);
      if (gq < hi_u) {
        v[q] = TO_BOX ? ld_cg16(lin + (gq << 4)) : *reinterpret_cast<const uint4*>(addr[q]);
        cursor_step(x, c, kBoxThreads);
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const unsigned long long gq = g + (unsigned long long)q * kBoxThreads;
      if (gq < hi_u) {
        if (TO_BOX) *reinterpret_cast<uint4*>(addr[q]) = v[q];
        else *reinterpret_cast<uint4*>(lin + (gq << 4)) = v[q];
      }
    }
  }
}

// The same for units of 1, 2, 4 or 8 bytes (U = an unsigned integer type of that size): eight units per
// thread in flight, which is what a gather of single elements along a strided direction needs.
template <typename U, bool TO_BOX>
__device__ __forceinline__ void copy_small(const Box& x, char* lin, unsigned long long lo_u, unsigned long long hi_u) {
  unsigned long long g = lo_u + threadIdx.x;
  if (g >= hi_u) return;
  Cursor c = cursor_at(x, g);
  for (; g < hi_u; g += 8ull * kBoxThreads) {
    U v[8];
    char* addr[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const unsigned long long gq = g + (unsigned long long)q * kBoxThreads;
      addr[q] = c.rowp + (size_t)c.col * sizeof(U);
      if (gq < hi_u) {
        v[q] = TO_BOX ? *reinterpret_cast<const volatile U*>(lin + gq * sizeof(U)) : *reinterpret_cast<const U*>(addr[q]);
        cursor_step(x, c, kBoxThreads);
      }
    }
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const unsigned long long gq = g + (unsigned long long)q * kBoxThreads;
      if (gq < hi_u) {
        if (TO_BOX) *reinterpret_cast<U*>(addr[q]) = v[q];
        else *reinterpret_cast<U*>(lin + gq * sizeof(U)) = v[q];
      }
    }
  }
}
template <bool TO_BOX>
__device__ __forceinline__ void copy_small_any(const Box& x, int unit, char* lin, unsigned long long lo_u,
                                               unsigned long long hi_u) {
  switch (unit) {
    case 1: copy_small<uint8_t, TO_BOX>(x, lin, lo_u, hi_u); break;
    case 2: copy_small<uint16_t, TO_BOX>(x, lin, lo_u, hi_u); break;
    case 4: copy_small<uint32_t, TO_BOX>(x, lin, lo_u, hi_u); break;
    default: copy_small<uint64_t, TO_BOX>(x, lin, lo_u, hi_u); break;
  }
}

// Thread 0 waits (bounded) until the counter at p has reached `want`; every thread of the CTA
// learns the outcome.  SYS: the counter is written by another GPU.
template <bool SYS>
__device__ bool cta_wait(const uint32_t* p, uint32_t want, StatusRecord* st, int where, int* sh_fail) {
  if (threadIdx.x == 0) {
    uint32_t seen = SYS ? ld_acquire_sys_u32(p) : ld_acquire_gpu_u32(p);
    if ((int32_t)(seen - want) < 0) {
      const uint64_t t0 = globaltimer_ns();
      uint32_t it = 0;
      while (true) {
        seen = SYS ? ld_acquire_sys_u32(p) : ld_acquire_gpu_u32(p);
        if ((int32_t)(seen - want) >= 0) break;
        if ((++it & 0x3f) == 0) {
          if (st != nullptr && *reinterpret_cast<volatile int*>(&st->code) != 0) { *sh_fail = 1; break; }
          if (globaltimer_ns() - t0 > kSpinLimitNs) {
            report_timeout(st, where, (int)want, (int)seen);
            *sh_fail = 1;
            break;
          }
        }
      }
      if (SYS && blockIdx.x == 0) account_wait(st, 5, globaltimer_ns() - t0);
    }
  }
  __syncthreads();
  return *sh_fail == 0;
}

__global__ void __launch_bounds__(kBoxThreads) box_exchange_kernel(const __grid_constant__ BoxArgs A) {
  __shared__ int fail;
  if (threadIdx.x == 0) fail = 0;
  __syncthreads();
  const int half = gridDim.x / 2;
  const bool sender = (int)blockIdx.x < half;        // local copies count as sends
  const int my = sender ? blockIdx.x : blockIdx.x - half;
  for (int it = 0; it < A.n_items; ++it) {
    const BoxItem& m = A.item[it];
    if ((m.kind == kRecv) == sender) continue;
    // The CTAs of a role are dealt out to the items of the current phase, so that a CTA never
    // serves two pairs in one phase: a pair's chunks then depend on that pair's CTAs only, and a
    // slow pair cannot hold up another one (no wait cycle through a shared CTA).
    int k = 0, j = 0;
    for (int o = 0; o < A.n_items; ++o) {
      const BoxItem& x = A.item[o];
      if ((x.kind == kRecv) == sender || x.phase != m.phase) continue;
      if (o < it) ++j;
      ++k;
    }
    if (my % k != j) continue;
    const int nserve = (half - j + k - 1) / k, mine = my / k;
    unsigned long long w = 0;                        // running index of this item's pieces
    const unsigned long long nchunks = m.kind == kLocal ? 1 : (m.bytes + A.chunk_bytes - 1) / A.chunk_bytes;
    for (unsigned long long c = 0; c < nchunks; ++c) {
      const unsigned long long c_lo = m.kind == kLocal ? 0 : c * A.chunk_bytes;
      const unsigned long long c_hi = m.kind == kLocal ? m.bytes : (c_lo + A.chunk_bytes < m.bytes ? c_lo + A.chunk_bytes : m.bytes);
      const unsigned long long kPieceBytes = piece_bytes_for(m.kind == kLocal ? (m.unit < m.unit_b ? m.unit : m.unit_b) : m.unit);
      const unsigned pieces = (unsigned)((c_hi - c_lo + kPieceBytes - 1) / kPieceBytes);
      const unsigned seq = m.first_seq + (unsigned)c;
      const int buf = seq % kBoxBufs;
      const unsigned use = seq / kBoxBufs;
      for (unsigned pc = 0; pc < pieces; ++pc, ++w) {
        if ((int)(w % (unsigned long long)nserve) != mine) continue;
        // everything of the phases before this one is complete on this GPU
        if (m.phase > 0 && !cta_wait<false>(A.progress, A.phase_target[m.phase - 1], A.status, 300 + m.phase, &fail))
          return;
        const unsigned long long lo = c_lo + (unsigned long long)pc * kPieceBytes;
        const unsigned long long hi = lo + kPieceBytes < c_hi ? lo + kPieceBytes : c_hi;
        if (m.kind == kSend) {
          if (!cta_wait<true>(A.pad[A.me] + PAD_BOX_CONSUMED + buf * 8 + m.peer, use, A.status, 310, &fail)) return;
          char* dst = A.inbox[m.peer] + (unsigned long long)A.me * A.slot_bytes + (unsigned long long)buf * A.chunk_bytes - c_lo;
          const int unit = m.unit;
          const bool clear = m.clear_source != 0;
          StatusRecord* st = A.status;
#ifndef DD_BOUNDS_CHECK
          if (unit == 16 && !clear) {
            copy16_rows<false>(m.a, dst, lo / 16, hi / 16);
          } else if (unit != 16 && !clear) {
            copy_small_any<false>(m.a, unit, dst, lo / unit, hi / unit);
          } else
#endif
          {
            const Box& bx = m.a;
            walk_units(bx, unit, lo / unit, hi / unit, [&](char* src, unsigned long long g) {
              if (in_bounds(bx, src, unit, st, g)) move_unit(dst + g * unit, src, unit, kAddNone, clear);
            });
          }
        } else if (m.kind == kRecv) {
          if (!cta_wait<true>(A.pad[A.me] + PAD_BOX_DELIVERED + buf * 8 + m.peer, use + 1, A.status, 311, &fail)) return;
          char* src = A.inbox[A.me] + (unsigned long long)m.peer * A.slot_bytes + (unsigned long long)buf * A.chunk_bytes - c_lo;
          const int unit = m.unit, add = m.add;
          StatusRecord* st = A.status;
          const Box& bx = m.a;
#ifndef DD_BOUNDS_CHECK
          if (unit == 16 && add == kAddNone) {
            copy16_rows<true>(bx, src, lo / 16, hi / 16);
          } else if (unit != 16 && add == kAddNone) {
            copy_small_any<true>(bx, unit, src, lo / unit, hi / unit);
          } else
#endif
          if (unit == 16) {
            walk_units(bx, 16, lo / 16, hi / 16, [&](char* to, unsigned long long g) {
              uint4 v = ld_cg16(src + g * 16);
              if (in_bounds(bx, to, 16, st, g)) move_unit(to, reinterpret_cast<char*>(&v), 16, add, false);
            });
          } else {
            walk_units(bx, unit, lo / unit, hi / unit, [&](char* to, unsigned long long g) {
              // (volatile read: the buffer was written by another GPU)
              uint64_t v = 0;
              const char* sp = src + g * unit;
              switch (unit) {
                case 1: v = *reinterpret_cast<const volatile uint8_t*>(sp); break;
                case 2: v = *reinterpret_cast<const volatile uint16_t*>(sp); break;
                case 4: v = *reinterpret_cast<const volatile uint32_t*>(sp); break;
                default: v = *reinterpret_cast<const volatile uint64_t*>(sp); break;
              }
              if (in_bounds(bx, to, unit, st, g)) move_unit(to, reinterpret_cast<char*>(&v), unit, add, false);
            });
          }
        } else {
          // local copy: the two sides may have different units; walk in the smaller one
          const int unit = m.unit < m.unit_b ? m.unit : m.unit_b;
          const int ra = m.unit / unit, rb = m.unit_b / unit;
          StatusRecord* st = A.status;
          const Box& ba = m.a;
          const Box& bb = m.b;
          if (ra == 1 && rb == 1) {
            // the same unit on both sides: one cursor per box, stepped together
            unsigned long long g = lo / unit + threadIdx.x;
            const unsigned long long g_end = hi / unit;
            if (g < g_end) {
              Cursor ca = cursor_at(ba, g), cb = cursor_at(bb, g);
              for (; g < g_end; g += kBoxThreads) {
                char* from = ca.rowp + (size_t)ca.col * unit;
                char* to = cb.rowp + (size_t)cb.col * unit;
                if (in_bounds(bb, to, unit, st, g) && in_bounds(ba, from, unit, st, g))
                  move_unit(to, from, unit, kAddNone, false);
                cursor_step(ba, ca, kBoxThreads);
                cursor_step(bb, cb, kBoxThreads);
              }
            }
          } else {
            for (unsigned long long g = lo / unit + threadIdx.x; g < hi / unit; g += kBoxThreads) {
              char* to = unit_addr(bb, m.unit_b, g / rb) + (g % rb) * unit;
              char* from = unit_addr(ba, m.unit, g / ra) + (g % ra) * unit;
              if (in_bounds(bb, to, unit, st, g) && in_bounds(ba, from, unit, st, g))
                move_unit(to, from, unit, kAddNone, false);
            }
          }
        }
        // the piece is done; whoever completes the chunk signals the other GPU
        __syncthreads();
        if (threadIdx.x == 0) {
          if (m.kind != kLocal) {
            __threadfence_system();
            unsigned* cnt = A.piece_count + ((m.kind == kSend ? 0 : 1) * kMaxPeers + m.peer) * kBoxBufs + buf;
            const unsigned old = atomicAdd(cnt, 1u);
            if (old == pieces - 1) {
              atomicExch(cnt, 0u);
              __threadfence_system();
              if (m.kind == kSend) red_release_sys_u32(A.pad[m.peer] + PAD_BOX_DELIVERED + buf * 8 + A.me);
              else red_release_sys_u32(A.pad[m.peer] + PAD_BOX_CONSUMED + buf * 8 + A.me);
            }
          } else {
            __threadfence();
          }
          atomicAdd(A.progress, 1u);
        }
        __syncthreads();
      }
    }
  }
}

unsigned* g_box_scratch[64] = {nullptr};   // per device: [0] progress, [16..] piece counters

}  // namespace

#ifdef DD_BOUNDS_CHECK
DD_API int dd_bounds_checked() { return 1; }
#else
DD_API int dd_bounds_checked() { return 0; }
#endif
DD_API int dd_box_max_items() { return kBoxMaxItems; }
DD_API int dd_box_bufs() { return kBoxBufs; }
DD_API int dd_box_piece_bytes(int unit) { return (int)piece_bytes_for(unit); }
DD_API int dd_box_item_bytes() { return (int)sizeof(BoxItem); }

// items: n_items BoxItem records in the layout of this file (see parallel/box_exchange.py);
// inbox / pads: 8 pointers each, by world rank (null where there is no such rank).
// phase_target[p]: value of the local progress counter when phase p is complete.
DD_API int dd_box_exchange(const void* items, int n_items, int n_phases, const unsigned* phase_target,
                           void* const* inbox, void* const* pads, int me, unsigned long long slot_bytes,
                           unsigned long long chunk_bytes, void* stream) {
  if (n_items < 0 || n_items > kBoxMaxItems || n_phases < 1 || n_phases > 8 || me < 0 || me >= kMaxPeers)
    return DD_ERR_BAD_ARG;
  if (chunk_bytes == 0 || chunk_bytes % 16 || chunk_bytes * kBoxBufs > slot_bytes) return DD_ERR_BAD_ARG;
  if (n_items == 0) return DD_OK;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return DD_ERR_BAD_ARG;
  if (g_box_scratch[dev] == nullptr) {
    unsigned* p = nullptr;
    e = cudaMalloc(&p, 4096);
    if (e != cudaSuccess) return (int)e;
    e = cudaMemset(p, 0, 4096);
    if (e != cudaSuccess) return (int)e;
    g_box_scratch[dev] = p;
  }
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  static BoxArgs a;     // (large: kept off the stack; the launch copies it)
  memcpy(a.item, items, sizeof(BoxItem) * (size_t)n_items);
  a.n_items = n_items;
  a.n_phases = n_phases;
  for (int p = 0; p < 8; ++p) a.phase_target[p] = p < n_phases ? phase_target[p] : 0;
  a.progress = g_box_scratch[dev];
  a.piece_count = g_box_scratch[dev] + 16;
  for (int r = 0; r < kMaxPeers; ++r) {
    a.inbox[r] = reinterpret_cast<char*>(inbox[r]);
    a.pad[r] = reinterpret_cast<uint32_t*>(pads[r]);
  }
  a.me = me;
  a.slot_bytes = slot_bytes;
  a.chunk_bytes = chunk_bytes;
  for (int i = 0; i < n_items; ++i) {
    const BoxItem& m = a.item[i];
    if (m.kind < kSend || m.kind > kLocal || m.phase < 0 || m.phase >= n_phases) return DD_ERR_BAD_ARG;
    if (m.unit != 1 && m.unit != 2 && m.unit != 4 && m.unit != 8 && m.unit != 16) return DD_ERR_BAD_ARG;
    if (m.bytes == 0 || m.bytes % m.unit) return DD_ERR_BAD_ARG;
    if (m.kind != kLocal && (m.peer < 0 || m.peer >= kMaxPeers || m.peer == me || inbox[m.peer] == nullptr))
      return DD_ERR_BAD_ARG;
    if (i > 0 && m.phase < a.item[i - 1].phase) return DD_ERR_BAD_ARG;     // items come sorted by phase
  }
  for (int p = 0; p < n_phases; ++p) {
    int ns = 0, nr = 0;
    for (int i = 0; i < n_items; ++i)
      if (a.item[i].phase == p) (a.item[i].kind == kRecv ? nr : ns)++;
    if (ns > kBoxCtas / 2 || nr > kBoxCtas / 2) return DD_ERR_TOO_LARGE;
  }
  int err = 0;
  a.status = device_status(&err);
  if (err) return err;
  box_exchange_kernel<<<kBoxCtas, kBoxThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

// The progress counter's current value on this device (0 before the first exchange): read
// with a device synchronisation, for tests and to start the host's bookkeeping.
DD_API int dd_box_progress(unsigned* out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DD_ERR_BAD_ARG;
  *out = 0;
  if (g_box_scratch[dev] == nullptr) return DD_OK;
  return (int)cudaMemcpy(out, g_box_scratch[dev], sizeof(unsigned), cudaMemcpyDeviceToHost);
}

// The same index arithmetic on the host, for tests without a GPU: moves the units
// [0, bytes / unit) of box `a` of a send item into a contiguous buffer (kind 0), from a
// contiguous buffer into box `a` of a recv item (kind 1), or box a -> box b (kind 2).
DD_API int dd_box_copy_host(const void* item, void* contiguous) {
  BoxItem m;
  memcpy(&m, item, sizeof(BoxItem));
  char* buf = reinterpret_cast<char*>(contiguous);
  if (m.kind == kSend) {
    for (unsigned long long g = 0; g < m.bytes / m.unit; ++g)
      move_unit(buf + g * m.unit, unit_addr(m.a, m.unit, g), m.unit, kAddNone, m.clear_source != 0);
  } else if (m.kind == kRecv) {
    if (m.add == kAddBF16 || m.add == kAddF16) return DD_ERR_BAD_ARG;     // (no host arithmetic for these)
    for (unsigned long long g = 0; g < m.bytes / m.unit; ++g)
      move_unit(unit_addr(m.a, m.unit, g), buf + g * m.unit, m.unit, m.add, false);
  } else {
    const int unit = m.unit < m.unit_b ? m.unit : m.unit_b;
    const int ra = m.unit / unit, rb = m.unit_b / unit;
    for (unsigned long long g = 0; g < m.bytes / unit; ++g)
      move_unit(unit_addr(m.b, m.unit_b, g / rb) + (g % rb) * unit, unit_addr(m.a, m.unit, g / ra) + (g % ra) * unit,
                unit, kAddNone, false);
  }
  return DD_OK;
}
