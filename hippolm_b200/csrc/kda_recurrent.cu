// Token-recurrent KDA forward (``kda_mode: fused_recurrent``; decode / inference: no backward).
//
// Per token t of a sequence, with the state h[K][V] in fp32:
//     h    *= exp(g[t])[:, None]
//     vp    = beta[t] * (v[t] - h^T k[t])
//     h    += k[t] (x) vp
//     o[t]  = h^T q[t]                 (q already scaled and, like k, already normalised)
// which is the recurrence of fla/ops/kda/fused_recurrent.py:145-190 of the reference.
//
// One CTA owns (sequence, head, 32 value columns): 256 threads = 8 warps, warp w holds K/8 consecutive key rows of the
// state in registers, lane = value column. The two reductions over K per token (h^T k and h^T q) are a register partial
// sum per warp plus an 8-way sum through shared memory. Inputs of the next token are prefetched into registers while the
// current one is reduced. Memory traffic is the algorithmic minimum: every q/k/v/g element is read once, o written once.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace hippo {
typedef __nv_bfloat16 bf16;

template <int DK>
__global__ void __launch_bounds__(256) kda_recurrent_fwd_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, const float* __restrict__ g,
    const float* __restrict__ beta, const int* __restrict__ cu, int H, const float* __restrict__ h0,
    bf16* __restrict__ o, float* __restrict__ fin) {
  constexpr int VS = 32, NW = 8, R = DK / NW;            // R key rows per warp
  const int n = blockIdx.z, hd = blockIdx.y, v0 = blockIdx.x * VS;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = cu[n], t1 = cu[n + 1];
  __shared__ float red[2][NW][VS];
  __shared__ float kq[2][3][DK];                         // double-buffered k, q, exp(g) of one token

  float h[R];
  const size_t sbase = (((size_t)n * H + hd) * DK) * DK;
#pragma unroll
  for (int r = 0; r < R; ++r) h[r] = h0 ? h0[sbase + (size_t)(warp * R + r) * DK + v0 + lane] : 0.f;

  auto stage = [&](int t, int buf) {
    const size_t base = ((size_t)t * H + hd) * DK;
    for (int i = threadIdx.x; i < DK; i += 256) {
      kq[buf][0][i] = __bfloat162float(k[base + i]);
      kq[buf][1][i] = __bfloat162float(q[base + i]);
      kq[buf][2][i] = __expf(g[base + i]);
    }
  };
  if (t0 < t1) stage(t0, 0);
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const int buf = (t - t0) & 1;
    const size_t base = ((size_t)t * H + hd) * DK;
    const float vt = __bfloat162float(v[base + v0 + lane]);
    const float bt = beta[(size_t)t * H + hd];
    if (t + 1 < t1) stage(t + 1, buf ^ 1);               // the other buffer was last read two barriers ago
    float part = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      h[r] *= kq[buf][2][warp * R + r];
      part += h[r] * kq[buf][0][warp * R + r];
    }
    red[0][warp][lane] = part;
    __syncthreads();
    float kv = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) kv += red[0][w][lane];
    const float vp = bt * (vt - kv);
    float po = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      h[r] += kq[buf][0][warp * R + r] * vp;
      po += h[r] * kq[buf][1][warp * R + r];
    }
    red[1][warp][lane] = po;
    __syncthreads();
    if (warp == 0) {
      float ot = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) ot += red[1][w][lane];
      o[base + v0 + lane] = __float2bfloat16(ot);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) fin[sbase + (size_t)(warp * R + r) * DK + v0 + lane] = h[r];
}
}  // namespace hippo

using namespace hippo;

// q, k, v: [T, H, DK] bf16; g: [T, H, DK] fp32 log decay; beta: [T, H] fp32; cu: [N + 1] int32 sequence offsets;
// h0: [N, H, DK, DK] fp32 or null; o: [T, H, DK] bf16; fin: [N, H, DK, DK] fp32.
extern "C" int hippo_kda_recurrent_fwd(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                       const int* cu, int N, int H, int DK, const float* h0, void* o, float* fin,
                                       void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (N <= 0 || H <= 0) return 0;
  dim3 grid(DK / 32, H, N);
  if (DK == 128)
    kda_recurrent_fwd_kernel<128><<<grid, 256, 0, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, g, beta, cu, H, h0,
                                                       (bf16*)o, fin);
  else if (DK == 64)
    kda_recurrent_fwd_kernel<64><<<grid, 256, 0, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, g, beta, cu, H, h0,
                                                      (bf16*)o, fin);
  else
    return -1;
  return (int)cudaGetLastError();
}
