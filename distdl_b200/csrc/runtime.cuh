// Host-side runtime shared by all entry points: per-device status record,
// driver entry points resolved at run time (no link-time libcuda dependency),
// tensor-map cache.
#pragma once

#include <cudaTypedefs.h>

#include "common.cuh"

namespace dd {

// Device pointer to this device's status record (allocated on first use).
StatusRecord* device_status(int* err);

// cuTensorMapEncodeTiled resolved through the runtime.
PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder();

// Encodes (or fetches from a small cache) a rank-3 bf16 tensor map with a
// 128-byte swizzle: dims {inner, outer, batch}, strides in BYTES for outer
// and batch, box {box_inner, box_outer, 1}.  Returns 0 on success.
int get_tensor_map_bf16_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                           uint64_t batch, uint64_t outer_stride_bytes, uint64_t batch_stride_bytes,
                           uint32_t box_inner, uint32_t box_outer);

// The same for fp32 elements (outputs written or reduced by TMA).
int get_tensor_map_f32_3d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                          uint64_t batch, uint64_t outer_stride_bytes, uint64_t batch_stride_bytes,
                          uint32_t box_inner, uint32_t box_outer);

int current_sm_count();

}  // namespace dd
