// NVLink multicast ("NVLS") memory and the all-reduce kernels that use it.
//
// A multicast object spans the GPUs of the job; every GPU binds one physical
// allocation of the same size to it.  Through the multicast mapping, one
// `multimem.ld_reduce` returns the SUM of the word at that offset over all bound
// GPUs (the addition happens inside NVSwitch) and one `multimem.st` writes a word
// into every GPU's copy.  An all-reduce then moves each byte over a GPU's links
// once in each direction instead of P - 1 times:
//   one shot  (small messages): every GPU ld_reduces the whole vector into its output;
//   two shots (large messages): GPU r ld_reduces slice r and multimem.st's the sums
//                               into every GPU's result buffer.
// The reference calls ncclAllReduce here
// (src/distdl/backends/nccl_cupy/functional/all_sum_reduce.py:73-76); NCCL picks its
// own NVLS algorithm inside.  Only ever local memory and this multicast mapping are
// touched: no TMA, no cluster multicast.
//
// Set-up is split between this file (driver calls, resolved at run time) and the
// host program, which has to carry the multicast object's file descriptor from the
// process that created it to the others (parallel/symm.py does that over a unix
// socket).  Barriers reuse the signal pads and counter flags of collectives.cu.
#include <unistd.h>

#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "runtime.cuh"

using namespace dd;

namespace {

template <typename F>
F driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return reinterpret_cast<F>(p);
}

struct Drv {
  PFN_cuMemCreate_v10020 mem_create;
  PFN_cuMemRelease_v10020 mem_release;
  PFN_cuMemAddressReserve_v10020 addr_reserve;
  PFN_cuMemAddressFree_v10020 addr_free;
  PFN_cuMemMap_v10020 mem_map;
  PFN_cuMemUnmap_v10020 mem_unmap;
  PFN_cuMemSetAccess_v10020 set_access;
  PFN_cuMemExportToShareableHandle_v10020 export_handle;
  PFN_cuMemImportFromShareableHandle_v10020 import_handle;
  PFN_cuMulticastCreate_v12010 mc_create;
  PFN_cuMulticastAddDevice_v12010 mc_add_device;
  PFN_cuMulticastBindMem_v12010 mc_bind_mem;
  PFN_cuMulticastUnbind_v12010 mc_unbind;
  PFN_cuMulticastGetGranularity_v12010 mc_granularity;
  bool ok;
};

const Drv& drv() {
  static Drv d = [] {
    Drv x;
    x.mem_create = driver_fn<PFN_cuMemCreate_v10020>("cuMemCreate");
    x.mem_release = driver_fn<PFN_cuMemRelease_v10020>("cuMemRelease");
    x.addr_reserve = driver_fn<PFN_cuMemAddressReserve_v10020>("cuMemAddressReserve");
    x.addr_free = driver_fn<PFN_cuMemAddressFree_v10020>("cuMemAddressFree");
    x.mem_map = driver_fn<PFN_cuMemMap_v10020>("cuMemMap");
    x.mem_unmap = driver_fn<PFN_cuMemUnmap_v10020>("cuMemUnmap");
    x.set_access = driver_fn<PFN_cuMemSetAccess_v10020>("cuMemSetAccess");
    x.export_handle = driver_fn<PFN_cuMemExportToShareableHandle_v10020>("cuMemExportToShareableHandle");
    x.import_handle = driver_fn<PFN_cuMemImportFromShareableHandle_v10020>("cuMemImportFromShareableHandle");
    x.mc_create = driver_fn<PFN_cuMulticastCreate_v12010>("cuMulticastCreate");
    x.mc_add_device = driver_fn<PFN_cuMulticastAddDevice_v12010>("cuMulticastAddDevice");
    x.mc_bind_mem = driver_fn<PFN_cuMulticastBindMem_v12010>("cuMulticastBindMem");
    x.mc_unbind = driver_fn<PFN_cuMulticastUnbind_v12010>("cuMulticastUnbind");
    x.mc_granularity = driver_fn<PFN_cuMulticastGetGranularity_v12010>("cuMulticastGetGranularity");
    x.ok = x.mem_create && x.mem_release && x.addr_reserve && x.addr_free && x.mem_map && x.mem_unmap &&
           x.set_access && x.export_handle && x.import_handle && x.mc_create && x.mc_add_device && x.mc_bind_mem &&
           x.mc_unbind && x.mc_granularity;
    return x;
  }();
  return d;
}

// One multicast region per process (the job-wide team).
struct McState {
  CUmemGenericAllocationHandle mc = 0, mem = 0;
  CUdeviceptr uc_va = 0, mc_va = 0;
  size_t size = 0;
  int dev = -1, n_devices = 0;
  bool bound = false;
} g_mc;

#define DRV_CHECK(call, what)                                                              \
  do {                                                                                     \
    CUresult r_ = (call);                                                                  \
    if (r_ != CUDA_SUCCESS) {                                                              \
      fprintf(stderr, "distdl_b200 multicast: %s failed with CUresult %d\n", what, (int)r_); \
      return DD_ERR_DRIVER;                                                                \
    }                                                                                      \
  } while (0)

CUmulticastObjectProp mc_prop(int n_devices, size_t size) {
  CUmulticastObjectProp p;
  memset(&p, 0, sizeof(p));
  p.numDevices = (unsigned)n_devices;
  p.size = size;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

}  // namespace

// 1 when the device and driver support multicast objects, else 0.
DD_API int dd_mc_supported() {
  if (!drv().ok) return 0;
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  auto get_attr = driver_fn<PFN_cuDeviceGetAttribute_v2000>("cuDeviceGetAttribute");
  if (get_attr == nullptr) return 0;
  cudaFree(nullptr);
  if (get_attr(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, (CUdevice)dev) != CUDA_SUCCESS) return 0;
  return v ? 1 : 0;
}

// Size rounded up to the multicast granularity of an n-device object.
DD_API int dd_mc_round_size(int n_devices, size_t bytes, size_t* out) {
  if (!drv().ok) return DD_ERR_DRIVER;
  CUmulticastObjectProp p = mc_prop(n_devices, bytes);
  size_t g = 0;
  DRV_CHECK(drv().mc_granularity(&g, &p, CU_MULTICAST_GRANULARITY_RECOMMENDED), "cuMulticastGetGranularity");
  *out = (bytes + g - 1) / g * g;
  return DD_OK;
}

// The creating process: makes the object and exports it as a file descriptor.
DD_API int dd_mc_create(int n_devices, size_t size, int* fd_out) {
  if (!drv().ok) return DD_ERR_DRIVER;
  if (g_mc.mc != 0) return DD_ERR_BAD_ARG;
  cudaFree(nullptr);
  CUmulticastObjectProp p = mc_prop(n_devices, size);
  DRV_CHECK(drv().mc_create(&g_mc.mc, &p), "cuMulticastCreate");
  int fd = -1;
  DRV_CHECK(drv().export_handle(&fd, g_mc.mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
            "cuMemExportToShareableHandle");
  *fd_out = fd;
  g_mc.size = size;
  g_mc.n_devices = n_devices;
  return DD_OK;
}

// Every other process: imports the object from the descriptor it was handed.
DD_API int dd_mc_import(int n_devices, size_t size, int fd) {
  if (!drv().ok) return DD_ERR_DRIVER;
  if (g_mc.mc != 0) return DD_ERR_BAD_ARG;
  cudaFree(nullptr);
  DRV_CHECK(drv().import_handle(&g_mc.mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
            "cuMemImportFromShareableHandle");
  g_mc.size = size;
  g_mc.n_devices = n_devices;
  return DD_OK;
}

// Every process, after all have the object: adds its own device.
DD_API int dd_mc_add_device() {
  if (g_mc.mc == 0) return DD_ERR_BAD_ARG;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return DD_ERR_DRIVER;
  g_mc.dev = dev;
  DRV_CHECK(drv().mc_add_device(g_mc.mc, (CUdevice)dev), "cuMulticastAddDevice");
  return DD_OK;
}

// Every process, after all devices were added: allocates its physical memory, binds it to
// the object and maps both views.  *local = this GPU's copy, *multicast = the multicast view.
DD_API int dd_mc_bind_and_map(void** local, void** multicast) {
  if (g_mc.mc == 0 || g_mc.dev < 0 || g_mc.bound) return DD_ERR_BAD_ARG;
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = g_mc.dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  DRV_CHECK(drv().mem_create(&g_mc.mem, g_mc.size, &prop, 0), "cuMemCreate");
  DRV_CHECK(drv().mc_bind_mem(g_mc.mc, 0, g_mc.mem, 0, g_mc.size, 0), "cuMulticastBindMem");
  g_mc.bound = true;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = g_mc.dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  DRV_CHECK(drv().addr_reserve(&g_mc.uc_va, g_mc.size, 0, 0, 0), "cuMemAddressReserve");
  DRV_CHECK(drv().mem_map(g_mc.uc_va, g_mc.size, 0, g_mc.mem, 0), "cuMemMap");
  DRV_CHECK(drv().set_access(g_mc.uc_va, g_mc.size, &acc, 1), "cuMemSetAccess");
  DRV_CHECK(drv().addr_reserve(&g_mc.mc_va, g_mc.size, 0, 0, 0), "cuMemAddressReserve (multicast)");
  DRV_CHECK(drv().mem_map(g_mc.mc_va, g_mc.size, 0, g_mc.mc, 0), "cuMemMap (multicast)");
  DRV_CHECK(drv().set_access(g_mc.mc_va, g_mc.size, &acc, 1), "cuMemSetAccess (multicast)");
  if (cudaMemset(reinterpret_cast<void*>(g_mc.uc_va), 0, g_mc.size) != cudaSuccess) return DD_ERR_DRIVER;
  *local = reinterpret_cast<void*>(g_mc.uc_va);
  *multicast = reinterpret_cast<void*>(g_mc.mc_va);
  return DD_OK;
}

// Every process, when no kernel that uses the region is in flight anywhere (the caller puts a
// host barrier before this): unmaps, unbinds and releases.  After it the region is gone.
DD_API int dd_mc_teardown() {
  if (g_mc.mc == 0) return DD_OK;
  cudaDeviceSynchronize();
  if (g_mc.mc_va) { drv().mem_unmap(g_mc.mc_va, g_mc.size); drv().addr_free(g_mc.mc_va, g_mc.size); }
  if (g_mc.uc_va) { drv().mem_unmap(g_mc.uc_va, g_mc.size); drv().addr_free(g_mc.uc_va, g_mc.size); }
  if (g_mc.bound) drv().mc_unbind(g_mc.mc, (CUdevice)g_mc.dev, 0, g_mc.size);
  if (g_mc.mem) drv().mem_release(g_mc.mem);
  drv().mem_release(g_mc.mc);
  g_mc = McState();
  return DD_OK;
}

DD_API int dd_close_fd(int fd) { return close(fd); }

// ---------------------------------------------------------------------------
// Kernels
// ---------------------------------------------------------------------------
namespace {

constexpr int kMaxPeers = 8;
constexpr int kMcThreads = 512;
constexpr int kMcMaxCtas = 144;
// signal-pad words [1200, 1200 + 144 * 8): one counter per (CTA, writer) for these kernels
constexpr int PAD_MC = 1200;

struct McTeam {
  int n, me;                    // team = the whole job; me = my rank
  uint32_t* pad[kMaxPeers];     // signal pads (peer-mapped)
  uint32_t expect;              // value of every peer's counter at this launch's first barrier
  StatusRecord* status;
};

__device__ __forceinline__ uint4 multimem_ld_reduce_f32(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
// 16 bytes that another GPU wrote through the multicast mapping: read at L2
__device__ __forceinline__ uint4 ld_cg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void multimem_st(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// store(v, sum) for the vectors v = lo + tid, + stride, ... < hi, where sum is the job-wide sum of the
// 16-byte vector at byte offset `base + 16 v` of the multicast region; kMcDepth reductions per thread
// are in flight before the first store (the switch's round trip is a few microseconds).
constexpr int kMcDepth = 8;
template <bool BF16, typename Store>
__device__ __forceinline__ void mc_reduce_loop(const char* mc, size_t lo, size_t hi, size_t tid, size_t stride,
                                               Store store) {
  for (size_t v = lo + tid; v < hi; v += kMcDepth * stride) {
    uint4 r[kMcDepth];
#pragma unroll
    for (int q = 0; q < kMcDepth; ++q) {
      const size_t vq = v + q * stride;
      if (vq < hi) r[q] = BF16 ? multimem_ld_reduce_bf16(mc + (vq << 4)) : multimem_ld_reduce_f32(mc + (vq << 4));
    }
#pragma unroll
    for (int q = 0; q < kMcDepth; ++q) {
      const size_t vq = v + q * stride;
      if (vq < hi) store(vq, r[q]);
    }
  }
}

// Barrier number `step` of this launch between CTA blockIdx.x of all GPUs (counters only
// grow; bounded wait).  Returns false after a time-out.
__device__ bool mc_barrier(const McTeam& t, uint32_t step, int* sh_fail) {
  __syncthreads();
  if (threadIdx.x < t.n && (int)threadIdx.x != t.me) {
    const int i = threadIdx.x;
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(t.pad[i] + PAD_MC + blockIdx.x * kMaxPeers + t.me)
                 : "memory");
    const uint32_t want = t.expect + step;
    const uint32_t* mine = t.pad[t.me] + PAD_MC + blockIdx.x * kMaxPeers + i;
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0, seen;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if ((int32_t)(seen - want) >= 0) break;
      if ((++it & 0xff) == 0) {
        if (t.status != nullptr && *reinterpret_cast<volatile int*>(&t.status->code) != 0) { *sh_fail = 1; break; }
        if (globaltimer_ns() - t0 > kSpinLimitNs) {
          report_timeout(t.status, 400 + (int)step, (int)want, (int)seen);
          *sh_fail = 1;
          break;
        }
      }
    }
  }
  __syncthreads();
  return *sh_fail == 0;
}

// in_off / out_off: byte offsets inside the region.  Input of every GPU at [in_off, in_off + bytes)
// of its copy.  one_shot: result to `out` (ordinary local memory).  Otherwise the sums land at
// [out_off, out_off + bytes) of every GPU's copy and each GPU copies them to `out` afterwards.
template <bool BF16>
__global__ void __launch_bounds__(kMcThreads)
mc_allreduce_kernel(const McTeam t, char* mc_base, char* uc_base, size_t in_off, size_t out_off, char* out,
                    size_t bytes, int one_shot) {
  __shared__ int fail;
  if (threadIdx.x == 0) fail = 0;
  const size_t nvec = bytes >> 4;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  if (!mc_barrier(t, 0, &fail)) return;                 // every GPU's input is in place
  if (one_shot == 2) {
    // reduce-scatter: `bytes` is one member's slice; member i's slice is the i-th of every input
    const size_t base = in_off + (size_t)t.me * bytes;
    mc_reduce_loop<BF16>(mc_base + base, 0, nvec, tid, stride,
                         [&](size_t v, const uint4& r) { *reinterpret_cast<uint4*>(out + (v << 4)) = r; });
    mc_barrier(t, 1, &fail);
    return;
  }
  if (one_shot) {
    mc_reduce_loop<BF16>(mc_base + in_off, 0, nvec, tid, stride,
                         [&](size_t v, const uint4& r) { *reinterpret_cast<uint4*>(out + (v << 4)) = r; });
    mc_barrier(t, 1, &fail);                            // nobody overwrites its input before all have read
    return;
  }
  const size_t per = (nvec + t.n - 1) / t.n;
  const size_t lo = per * t.me, hi = lo + per < nvec ? lo + per : nvec;
  char* mc_out = mc_base + out_off;
  mc_reduce_loop<BF16>(mc_base + in_off, lo, hi, tid, stride,
                       [&](size_t v, const uint4& r) { multimem_st(mc_out + (v << 4), r); });
  if (!mc_barrier(t, 1, &fail)) return;                 // all slices have been written everywhere
  // The barrier pairs CTA b of this GPU with CTA b of every other GPU only: read, of every member's
  // slice, exactly the vectors that the same-numbered CTA of that member wrote.
  for (int i = 0; i < t.n; ++i) {
    const size_t lo_i = per * i, hi_i = lo_i + per < nvec ? lo_i + per : nvec;
    for (size_t v = lo_i + tid; v < hi_i; v += 4 * stride) {
      uint4 r[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (v + q * stride < hi_i) r[q] = ld_cg16(uc_base + out_off + ((v + q * stride) << 4));
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (v + q * stride < hi_i) *reinterpret_cast<uint4*>(out + ((v + q * stride) << 4)) = r[q];
    }
  }
}

}  // namespace

// dtype 0 = bf16, 1 = fp32; bytes a multiple of 16; the input must already be at in_off of this
// GPU's copy (written on `stream` before this call).  *steps = barrier steps consumed.
// one_shot: 1 = all-reduce read in one pass, 0 = all-reduce in two shots, 2 = reduce-scatter (the
// input holds n slices of `bytes` each, member i receives the sum of everybody's slice i).
DD_API int dd_mc_allreduce(int n, int me, void* const* pads, unsigned expect, size_t in_off, size_t out_off,
                           void* out, size_t bytes, int dtype, int one_shot, int ctas, int* steps, void* stream) {
  if (g_mc.mc_va == 0) return DD_ERR_BAD_ARG;
  if (n < 2 || n > kMaxPeers || me < 0 || me >= n || n != g_mc.n_devices) return DD_ERR_BAD_ARG;
  if (bytes % 16 || in_off % 16 || out_off % 16) return DD_ERR_ALIGN;
  if (one_shot == 2) {
    if (in_off + (size_t)n * bytes > g_mc.size) return DD_ERR_TOO_LARGE;
  } else if (in_off + bytes > g_mc.size || (!one_shot && out_off + bytes > g_mc.size)) {
    return DD_ERR_TOO_LARGE;
  }
  McTeam t;
  t.n = n; t.me = me; t.expect = expect;
  for (int i = 0; i < n; ++i) t.pad[i] = reinterpret_cast<uint32_t*>(pads[i]);
  int err = 0;
  t.status = device_status(&err);
  if (err) return err;
  // The caller passes the same grid at every launch of the process (and on every GPU): every CTA
  // owns one counter per peer, and the host counts barrier steps once for all of them, so all
  // slots have to advance in step from launch to launch.
  if (ctas < 1 || ctas > kMcMaxCtas) return DD_ERR_BAD_ARG;
  *steps = 2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  char* mc = reinterpret_cast<char*>(g_mc.mc_va);
  char* uc = reinterpret_cast<char*>(g_mc.uc_va);
  if (dtype == 0)
    mc_allreduce_kernel<true><<<ctas, kMcThreads, 0, s>>>(t, mc, uc, in_off, out_off, (char*)out, bytes, one_shot);
  else
    mc_allreduce_kernel<false><<<ctas, kMcThreads, 0, s>>>(t, mc, uc, in_off, out_off, (char*)out, bytes, one_shot);
  return (int)cudaGetLastError();
}
DD_API int dd_mc_max_ctas() { return kMcMaxCtas; }
