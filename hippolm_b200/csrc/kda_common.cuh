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
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---- mma.sync m16n8k16 (bf16 in, fp32 accumulate) and ldmatrix fragment loads
// C fragment: c0,c1 = (row g, cols 2t, 2t+1), c2,c3 = (row g+8, same cols) with g = lane >> 2, t = lane & 3
__device__ __forceinline__ void kda_ldsm_x4(unsigned (&r)[4], const void* p) {
  unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void kda_ldsm_x4_t(unsigned (&r)[4], const void* p) {
  unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void kda_mma16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// A fragment (16 rows x 16 k) of a row-major [rows][ld] tile at (row0, k0)
__device__ __forceinline__ void kda_frag_a(unsigned (&r)[4], const bf16* tile, int ld, int row0, int k0, int lane) {
  kda_ldsm_x4(r, tile + (row0 + (lane & 15)) * ld + k0 + (lane >> 4) * 8);
}
// A fragment of the TRANSPOSE of a row-major [k][ld] tile: A[m][k] = tile[k0 + k][m0 + m]
__device__ __forceinline__ void kda_frag_a_t(unsigned (&r)[4], const bf16* tile, int ld, int m0, int k0, int lane) {
  kda_ldsm_x4_t(r, tile + (k0 + (lane & 7) + (lane >> 4) * 8) * ld + m0 + ((lane >> 3) & 1) * 8);
}
// B fragments of two adjacent n-tiles (16 k x 16 n) from a row-major [k][ld] tile (n contiguous):
// r[0], r[1] -> n-tile at n0, r[2], r[3] -> n-tile at n0 + 8
__device__ __forceinline__ void kda_frag_b2(unsigned (&r)[4], const bf16* tile, int ld, int k0, int n0, int lane) {
  kda_ldsm_x4_t(r, tile + (k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + n0 + (lane >> 4) * 8);
}
// B fragments of two adjacent n-tiles from a row-major [n][ld] tile (k contiguous, i.e. B^T is stored):
// r[0], r[1] -> n-tile at n0, r[2], r[3] -> n-tile at n0 + 8
__device__ __forceinline__ void kda_frag_bt2(unsigned (&r)[4], const bf16* tile, int ld, int n0, int k0, int lane) {
  kda_ldsm_x4(r, tile + (n0 + (lane & 7) + (lane >> 4) * 8) * ld + k0 + ((lane >> 3) & 1) * 8);
}
__device__ __forceinline__ unsigned kda_pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
}
