// Shared definitions of the chunked KDA kernels.
#pragma once
#include <cuda_bf16.h>
namespace hippo {
typedef __nv_bfloat16 bf16;
constexpr int KDA_CHUNK = 64;

// 16-byte asynchronous global -> shared copy; src_bytes = 0 writes zeros (masked rows)
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int src_bytes = 16) {
  unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
}
