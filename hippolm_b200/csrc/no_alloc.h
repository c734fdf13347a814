// RMSNorm backward without any device allocation.
//
// This entry point has no counterpart in the reference; it exists for callers of this library that
// are not allowed to call cudaMalloc (or anything that does so for them, torch's caching allocator
// included): for example code running inside a fixed memory budget that was carved up in advance, a
// plugin whose host application owns all device memory, or a latency-critical path where an allocation
// (and the device synchronisation cudaFree can imply) is not acceptable.
//
//   int hippo_rmsnorm_bwd_noalloc(x, w, dy, rstd, dx, dw, T, D, stream)
//     x, dy : [T, D] bf16      w : [D] bf16      rstd : [T] fp32 (saved by the forward)
//     dx    : [T, D] bf16 out  dw : [D] fp32 out
//   Same results as hippo_rmsnorm_bwd. The caller still provides every input and output; only the
//   intermediate per-block partial sums of dw are kept inside the library, in a fixed array of
//   148 x 8192 floats (4.6 MiB) that each GPU using the library holds until the process exits.
//
//   Limits and rules
//   * D must be a multiple of 8 and at most 8192; larger rows return -22 and launch nothing.
//   * The first call on a device looks up the device address of the built-in array (one
//     cudaGetSymbolAddress call, made with that device current). Make that first call outside of any
//     stream capture.
//   * All calls on one device share the array. It is fully rewritten by each call, so calls that run one
//     after the other on a stream need no clearing; calls that may overlap on the GPU (different
//     streams, no ordering between them) race on it and must be serialised by the caller.
//   * No cudaMalloc, cudaFree or allocating library routine is called. Returns 0 or a CUDA error code.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
int hippo_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx, float* dw,
                              long long T, int D, void* stream);
#ifdef __cplusplus
}
#endif
