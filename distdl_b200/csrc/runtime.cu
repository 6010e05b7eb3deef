// Host runtime of the native library: status record, driver entry points,
// tensor-map cache, version / capability queries.
#include "runtime.cuh"

#include <cstdio>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace dd {

namespace {
std::mutex g_mu;
constexpr int kMaxDevices = 64;
StatusRecord* g_status[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};

struct MapKey {
  const void* base;
  uint64_t inner, outer, batch, s1, s2;
  uint32_t b0, b1;
  int dev;
  int f32;
  bool operator==(const MapKey& o) const {
    return f32 == o.f32 && base == o.base && inner == o.inner && outer == o.outer && batch == o.batch && s1 == o.s1 &&
           s2 == o.s2 && b0 == o.b0 && b1 == o.b1 && dev == o.dev;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = reinterpret_cast<uint64_t>(k.base) * 0x9E3779B97F4A7C15ull;
    auto mix = [&h](uint64_t v) { h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2); };
    mix(k.inner); mix(k.outer); mix(k.batch); mix(k.s1); mix(k.s2); mix(k.b0); mix(k.b1); mix(k.dev); mix(k.f32);
    return (size_t)h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
}  // namespace

StatusRecord* device_status(int* err) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev >= kMaxDevices) { if (err) *err = (int)e; return nullptr; }
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status[dev] == nullptr) {
    StatusRecord* p = nullptr;
    e = cudaMalloc(&p, sizeof(StatusRecord));
    if (e != cudaSuccess) { if (err) *err = (int)e; return nullptr; }
    e = cudaMemset(p, 0, sizeof(StatusRecord));
    if (e != cudaSuccess) { if (err) *err = (int)e; return nullptr; }
    g_status[dev] = p;
  }
  if (err) *err = 0;
  return g_status[dev];
}

int current_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

namespace {
int get_tensor_map_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t batch,
                      uint64_t outer_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_inner,
                      uint32_t box_outer, int f32);
}
int get_tensor_map_bf16_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                           uint64_t batch, uint64_t outer_stride_bytes, uint64_t batch_stride_bytes,
                           uint32_t box_inner, uint32_t box_outer) {
  return get_tensor_map_3d(out, base, inner, outer, batch, outer_stride_bytes, batch_stride_bytes, box_inner,
                           box_outer, 0);
}
int get_tensor_map_f32_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                          uint64_t batch, uint64_t outer_stride_bytes, uint64_t batch_stride_bytes,
                          uint32_t box_inner, uint32_t box_outer) {
  return get_tensor_map_3d(out, base, inner, outer, batch, outer_stride_bytes, batch_stride_bytes, box_inner,
                           box_outer, 1);
}
namespace {
int get_tensor_map_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t batch,
                      uint64_t outer_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_inner,
                      uint32_t box_outer, int f32) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (outer_stride_bytes & 15) || (batch_stride_bytes & 15))
    return DD_ERR_ALIGN;
  int dev = 0;
  cudaGetDevice(&dev);
  MapKey key{base, inner, outer, batch, outer_stride_bytes, batch_stride_bytes, box_inner, box_outer, dev, f32};
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
  }
  auto enc = tensor_map_encoder();
  if (!enc) return DD_ERR_DRIVER;
  // Driver calls need the primary context current on the calling thread; a
  // thread that has only ever used the runtime lazily (e.g. an autograd worker)
  // may not have it bound yet.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaSetDevice(dev);
    cudaFree(nullptr);
    ctx_bound = true;
  }
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {outer_stride_bytes, batch_stride_bytes};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "distdl_b200: cuTensorMapEncodeTiled failed (%d): base=%p dims={%llu,%llu,%llu} strides={%llu,%llu} "
            "box={%u,%u,1}\n",
            (int)r, base, (unsigned long long)inner, (unsigned long long)outer, (unsigned long long)batch,
            (unsigned long long)outer_stride_bytes, (unsigned long long)batch_stride_bytes, box_inner, box_outer);
    return DD_ERR_DRIVER;
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_maps.size() > 65536) g_maps.clear();
    g_maps.emplace(key, *out);
  }
  return 0;
}
}  // namespace

}  // namespace dd

// Reads and clears the device status record of the current device.
// out[4] = {code, where, expected, seen}.  Synchronises the device.
DD_API int dd_read_status(int* out) {
  int err = 0;
  dd::StatusRecord* st = dd::device_status(&err);
  if (!st) return err ? err : DD_ERR_DRIVER;
  cudaError_t e = cudaMemcpy(out, st, 4 * sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(st, 0, 4 * sizeof(int));
  return (int)e;
}

// Reads (and clears) the per-kind totals of nanoseconds spent in cross-GPU waits.
DD_API int dd_read_wait_ns(unsigned long long* out) {
  int err = 0;
  dd::StatusRecord* st = dd::device_status(&err);
  if (!st) return err ? err : DD_ERR_DRIVER;
  cudaError_t e = cudaMemcpy(out, st->wait_ns, sizeof(st->wait_ns), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(st->wait_ns, 0, sizeof(st->wait_ns));
  return (int)e;
}

DD_API int dd_version() { return 100; }
DD_API int dd_sm_count() { return dd::current_sm_count(); }
