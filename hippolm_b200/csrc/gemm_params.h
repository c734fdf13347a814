// Parameters shared by the one-CTA and the CTA-pair bf16 GEMM kernels.
#pragma once
#include <cuda_runtime.h>

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
};

// CTA-pair (cta_group::2) kernel, defined in gemm_bf16_2sm.cu. layout: 0 NT, 1 NN, 2 TN, 3 TT.
int launch_gemm_2sm(const void* A, const void* B, int layout, long long lda, long long ldb, const GemmParams& p,
                    int max_ctas, cudaStream_t stream);
bool gemm_2sm_enabled();

}  // namespace hippo
