// Parameters shared by the one-CTA and the CTA-pair bf16 GEMM kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace hippo {

struct GemmParams {
  int M, N, K;
  void* C; long long ldc;
  int out_fp32;        // 0 = bf16, 1 = fp32
  int accumulate;      // C += result
  float alpha;
  const void* Cin;     // optional bf16 [M, ldcin] addend: C = alpha*A*B + beta*Cin (bf16 output only)
  long long ldcin; float beta;
  int tiles_m, tiles_n;
  int sym_lower;       // CTA-pair kernel: skip the 256x256 tiles above the diagonal (square symmetric output)
  int ksplit;          // CTA-pair kernel: > 1 = the contraction is cut into ksplit slices, work item = (tile, slice), slice s
                       // writes its fp32 partial product to C + s * M * ldc (C is then a [ksplit * M, ldc] fp32 workspace)
  // CTA-pair kernel, EPI_LCE mode (logits of the linear + cross-entropy head): besides the bf16 logits, the epilogue emits
  // the softmax statistics of every row of every 256-column tile, taken from the accumulator while it is in registers.
  float2* lce_part = nullptr;              // [tiles_n][M]: (max, sum of exp(z - max)) over the tile's columns of the bf16-rounded logits
  const long long* lce_target = nullptr;   // [M]: target column of the row in this GEMM's N range, or -1
  float* lce_tz = nullptr;                 // [M]: logit at the target column; written only for rows whose target is >= 0
};

#ifdef __CUDACC__
// Epilogue of one 32-column chunk of one accumulator row (thread = row): C = alpha*acc [+ C] [+ beta*Cin].
// The addends are fetched BEFORE the TMEM load is waited for (epi_prefetch), so a read-modify-write epilogue
// pays one memory latency per chunk instead of one per 16-byte piece.
struct EpiPrefetch { uint4 v[8]; };

__device__ __forceinline__ float2 epi_bf2(uint32_t u) {      // two packed bf16 -> two floats, register only
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}

__device__ __forceinline__ void epi_prefetch(const GemmParams& p, int row, int col0, EpiPrefetch& pre) {
  if (row >= p.M || col0 + 32 > p.N) return;                 // ragged chunks take the scalar path below
  if (p.out_fp32) {
    if (p.accumulate) {
      const uint4* src = (const uint4*)((const float*)p.C + (long long)row * p.ldc + col0);
#pragma unroll
      for (int j = 0; j < 8; ++j) pre.v[j] = src[j];
    }
  } else {
    if (p.accumulate) {
      const uint4* src = (const uint4*)((const __nv_bfloat16*)p.C + (long long)row * p.ldc + col0);
#pragma unroll
      for (int j = 0; j < 4; ++j) pre.v[j] = src[j];
    }
    if (p.Cin) {
      const uint4* src = (const uint4*)((const __nv_bfloat16*)p.Cin + (long long)row * p.ldcin + col0);
#pragma unroll
      for (int j = 0; j < 4; ++j) pre.v[4 + j] = src[j];
    }
  }
}

__device__ __forceinline__ void epi_store(const GemmParams& p, const uint32_t (&r)[32], int row, int col0,
                                          const EpiPrefetch& pre) {
  if (row >= p.M || col0 >= p.N) return;
  if (p.out_fp32) {
    float* crow = (float*)p.C + (long long)row * p.ldc + col0;
    if (col0 + 32 <= p.N) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 v = make_float4(__uint_as_float(r[4 * j]) * p.alpha, __uint_as_float(r[4 * j + 1]) * p.alpha,
                               __uint_as_float(r[4 * j + 2]) * p.alpha, __uint_as_float(r[4 * j + 3]) * p.alpha);
        if (p.accumulate) {
          v.x += __uint_as_float(pre.v[j].x); v.y += __uint_as_float(pre.v[j].y);
          v.z += __uint_as_float(pre.v[j].z); v.w += __uint_as_float(pre.v[j].w);
        }
        ((float4*)crow)[j] = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {                          // predicated, fully unrolled: r[] stays in registers
        if (col0 + j < p.N) {
          float v = __uint_as_float(r[j]) * p.alpha;
          if (p.accumulate) v += crow[j];
          crow[j] = v;
        }
      }
    }
  } else {
    __nv_bfloat16* crow = (__nv_bfloat16*)p.C + (long long)row * p.ldc + col0;
    if (col0 + 32 <= p.N) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * j + e]) * p.alpha;
        if (p.accumulate) {
          const uint32_t ow[4] = {pre.v[j].x, pre.v[j].y, pre.v[j].z, pre.v[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) { float2 of = epi_bf2(ow[e]); f[2 * e] += of.x; f[2 * e + 1] += of.y; }
        }
        if (p.Cin) {
          const uint32_t ow[4] = {pre.v[4 + j].x, pre.v[4 + j].y, pre.v[4 + j].z, pre.v[4 + j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) { float2 of = epi_bf2(ow[e]); f[2 * e] += p.beta * of.x; f[2 * e + 1] += p.beta * of.y; }
        }
        uint4 v;
        __nv_bfloat162* vb = (__nv_bfloat162*)&v;
#pragma unroll
        for (int e = 0; e < 4; ++e) vb[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        ((uint4*)crow)[j] = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (col0 + j < p.N) {
          float v = __uint_as_float(r[j]) * p.alpha;
          if (p.accumulate) v += __bfloat162float(crow[j]);
          if (p.Cin) v += p.beta * __bfloat162float(((const __nv_bfloat16*)p.Cin)[(long long)row * p.ldcin + col0 + j]);
          crow[j] = __float2bfloat16(v);
        }
      }
    }
  }
}
#endif  // __CUDACC__

// CTA-pair (cta_group::2) kernel, defined in gemm_bf16_2sm.cu. layout: 0 NT, 1 NN, 2 TN, 3 TT.
int launch_gemm_2sm(const void* A, const void* B, int layout, long long lda, long long ldb, const GemmParams& p,
                    int max_ctas, cudaStream_t stream);
bool gemm_2sm_enabled();

}  // namespace hippo
