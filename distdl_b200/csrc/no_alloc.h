// Entry point that allocates nothing.  It has no counterpart in the reference
// (microsoft/distdl has no native GPU code at all); it exists for users of this
// library who have to call into it from places where device memory cannot be
// allocated.
//
// Who needs it.  Some callers cannot call cudaMalloc when they need the
// operator: a plug-in or custom-call hook running inside a host program that
// reserved all device memory at start-up (a later cudaMalloc there fails), or a
// latency-critical section that cannot tolerate the implicit device-wide
// synchronisation of cudaMalloc / cudaFree.  The regular backward of the fused
// RMSNorm / LayerNorm (dd_norm_bwd) needs a scratch buffer for the per-CTA
// partial sums of the weight and bias gradients, which the caller normally
// allocates.  dd_norm_bwd_noalloc is the same computation with that scratch
// living in a fixed-size array inside the library.
//
// Contract.
//  * Inputs and outputs are passed by the caller exactly as for dd_norm_bwd
//    (dy, x, w, stats = per-row {mean, rstd} from the forward; dx, dw, db);
//    dw / db may be null.  No cudaMalloc, cudaFree or allocating library call
//    is made, by this function or on its behalf.
//  * dy, x, stats and dx must not be null (status 1001); dy, x, w and dx must be
//    16-byte aligned, stats 8-byte, dw and db 4-byte (status 1002).  These are
//    checked before anything is launched.
//  * Limit: d (row length) at most dd_norm_bwd_noalloc_max_d() = 8192 and a
//    multiple of 8; larger d is rejected with status 1003 and a message on
//    stderr.  The scratch takes dd_norm_bwd_noalloc_scratch_bytes() (9.25 MiB)
//    on every GPU that loads the library, from load until the process exits.
//  * The first call on a given device looks up the device address of the scratch
//    (cudaGetSymbolAddress, with that device current) and caches it; make that
//    first call before any stream capture is begun on that device.  The cache
//    is written without a lock; threads that race on a first call store the
//    same address, so the race is harmless.
//  * All calls on one device share the one scratch array, which keeps whatever
//    the previous call left in it.  Nothing in it has to start at zero (each
//    call overwrites every word it later reads), but two calls whose kernels
//    overlap on the GPU (different streams without ordering between them) race
//    on it: order such calls.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

int dd_norm_bwd_noalloc(int rms, const void* dy, const void* x, const void* w, const void* stats, void* dx,
                        float* dw, float* db, int accumulate, int rows, int d, void* stream);
int dd_norm_bwd_noalloc_max_d(void);
long long dd_norm_bwd_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
