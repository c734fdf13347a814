// Causal variable-length flash attention for the full-attention layers (forward + backward).
// Packed token-major q, k, v: [T, H, DH] bf16; documents given by a 64-row tile table
// (tile start, length, start of the tile's document). Online softmax in the exp2 domain, fp32
// accumulation, bf16 mma.sync m16n8k16 tiles fed by ldmatrix. Backward = row-dot preprocess,
// a dK/dV kernel (one CTA per key tile, warps own key rows) and a dQ kernel (one CTA per query tile,
// warps own query rows): no atomics, no cross-warp reductions, deterministic.
// The reference has no softmax-attention layer; this op exists for the hybrid 3:1 layer pattern.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace hippo {
typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int DH>
__device__ __forceinline__ void load_tile(bf16* dst, const bf16* src, int t0, int rows_valid, int H, int h, int tid,
                                          int nthreads) {
  constexpr int LD = DH + 8;
  for (int idx = tid; idx < 64 * (DH / 8); idx += nthreads) {
    int r = idx / (DH / 8), c8 = (idx % (DH / 8)) * 8;
    uint4 z = make_uint4(0, 0, 0, 0);
    if (r < rows_valid) z = *(const uint4*)(src + ((long long)(t0 + r) * H + h) * DH + c8);
    *(uint4*)(dst + r * LD + c8) = z;
  }
}

// A-operand fragments of a 16-row slab (row-major [rows][DH] in smem)
template <int DH>
__device__ __forceinline__ void load_a_frags(uint32_t (&f)[DH / 16][4], const bf16* base, int lane) {
  constexpr int LD = DH + 8;
#pragma unroll
  for (int kk = 0; kk < DH / 16; ++kk) ldsm_x4(f[kk], base + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
}

// S[16 x 64] = A(16 x DH) * Bt^T where Bt is [64][DH] row-major in smem (n = row of Bt, k = DH)
template <int DH>
__device__ __forceinline__ void mma_a_bt(float (&s)[8][4], const uint32_t (&af)[DH / 16][4], const bf16* Bt, int lane) {
  constexpr int LD = DH + 8;
#pragma unroll
  for (int n = 0; n < 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
#pragma unroll
  for (int kk = 0; kk < DH / 16; ++kk) {
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t b[4];
      ldsm_x4(b, Bt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
      mma16816(s[2 * np], af[kk], b[0], b[1]);
      mma16816(s[2 * np + 1], af[kk], b[2], b[3]);
    }
  }
}

// acc[16 x DH] += P(16 x 64, C-fragment layout) * B where B is [64][DH] row-major in smem (k = row, n = col)
template <int DH>
__device__ __forceinline__ void mma_p_b(float (&acc)[DH / 8][4], const float (&p)[8][4], const bf16* B, int lane) {
  constexpr int LD = DH + 8;
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < DH / 16; ++dp) {
      uint32_t b[4];
      ldsm_x4_t(b, B + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + dp * 16 + (lane >> 4) * 8);
      mma16816(acc[2 * dp], a, b[0], b[1]);
      mma16816(acc[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ forward
template <int DH>
__global__ void __launch_bounds__(128)
attn_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                const int* __restrict__ tile_start, const int* __restrict__ tile_len,
                const int* __restrict__ tile_seq0, int H, float scale_log2, bf16* __restrict__ o,
                float* __restrict__ lse) {
  constexpr int LD = DH + 8;
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* Qs = (bf16*)smem; bf16* Ks = Qs + 64 * LD; bf16* Vs = Ks + 64 * LD;
  const int tile = blockIdx.x, h = blockIdx.y;
  const int t0 = tile_start[tile], len = tile_len[tile], seq0 = tile_seq0[tile];
  if (len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  load_tile<DH>(Qs, q, t0, len, H, h, tid, 128);
  __syncthreads();
  uint32_t qf[DH / 16][4];
  load_a_frags<DH>(qf, Qs + warp * 16 * LD, lane);
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
  float oacc[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) { oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f; }
  const int nkv = (t0 - seq0) / 64 + 1;
  const int row0 = t0 + warp * 16 + g;                 // token index of this thread's first row
  for (int kt = 0; kt < nkv; ++kt) {
    const int kv0 = seq0 + kt * 64;
    const int kvlen = min(64, t0 + len - kv0);
    __syncthreads();
    load_tile<DH>(Ks, k, kv0, kvlen, H, h, tid, 128);
    load_tile<DH>(Vs, v, kv0, kvlen, H, h, tid, 128);
    __syncthreads();
    float s[8][4];
    mma_a_bt<DH>(s, qf, Ks, lane);
    const bool diag = (kt == nkv - 1);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float val = s[n][e] * scale_log2;
        if (diag) {
          int col = kv0 + n * 8 + 2 * tq + (e & 1);
          int row = row0 + (e >> 1) * 8;
          if (col > row) val = -INFINITY;
        }
        s[n][e] = val;
        mx[e >> 1] = fmaxf(mx[e >> 1], val);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xFFFFFFFFu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xFFFFFFFFu, mx[r], 2));
    }
    float alpha[2], rs[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mn = fmaxf(m_i[r], mx[r]);
      alpha[r] = (m_i[r] == -INFINITY) ? 0.f : exp2f(m_i[r] - mn);
      m_i[r] = mn;
    }
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float p = (m_i[e >> 1] == -INFINITY) ? 0.f : exp2f(s[n][e] - m_i[e >> 1]);
        s[n][e] = p; rs[e >> 1] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xFFFFFFFFu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xFFFFFFFFu, rs[r], 2);
      l_i[r] = l_i[r] * alpha[r] + rs[r];
    }
#pragma unroll
    for (int n = 0; n < DH / 8; ++n) { oacc[n][0] *= alpha[0]; oacc[n][1] *= alpha[0]; oacc[n][2] *= alpha[1]; oacc[n][3] *= alpha[1]; }
    mma_p_b<DH>(oacc, s, Vs, lane);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int rloc = warp * 16 + g + r * 8;
    if (rloc < len) {
      const float inv = l_i[r] > 0.f ? 1.f / l_i[r] : 0.f;
      const long long tok = t0 + rloc;
#pragma unroll
      for (int n = 0; n < DH / 8; ++n) {
        __nv_bfloat162 ov = __floats2bfloat162_rn(oacc[n][2 * r] * inv, oacc[n][2 * r + 1] * inv);
        *(__nv_bfloat162*)(o + (tok * H + h) * DH + n * 8 + 2 * tq) = ov;
      }
      if (tq == 0) lse[tok * H + h] = m_i[r] + log2f(l_i[r]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ backward
// delta[t,h] = sum_d dO * O
template <int DH>
__global__ void attn_bwd_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ d_o, float* __restrict__ delta,
                                      long long rows) {
  long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  int lane = threadIdx.x & 31;
  float s = 0.f;
  for (int c = lane * 2; c < DH; c += 64) {
    float2 a = __bfloat1622float2(*(const __nv_bfloat162*)(o + row * DH + c));
    float2 b = __bfloat1622float2(*(const __nv_bfloat162*)(d_o + row * DH + c));
    s += a.x * b.x + a.y * b.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
  if (lane == 0) delta[row] = s;
}

// dQ: one CTA per query tile, warps own 16 query rows, loop over key tiles
template <int DH>
__global__ void __launch_bounds__(128)
attn_bwd_dq_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                   const bf16* __restrict__ d_o, const float* __restrict__ lse, const float* __restrict__ delta,
                   const int* __restrict__ tile_start, const int* __restrict__ tile_len,
                   const int* __restrict__ tile_seq0, int H, float scale_log2, float scale, bf16* __restrict__ dq) {
  constexpr int LD = DH + 8;
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* Qs = (bf16*)smem; bf16* Ks = Qs + 64 * LD; bf16* Vs = Ks + 64 * LD; bf16* dOs = Vs + 64 * LD;
  const int tile = blockIdx.x, h = blockIdx.y;
  const int t0 = tile_start[tile], len = tile_len[tile], seq0 = tile_seq0[tile];
  if (len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  load_tile<DH>(Qs, q, t0, len, H, h, tid, 128);
  load_tile<DH>(dOs, d_o, t0, len, H, h, tid, 128);
  __syncthreads();
  uint32_t qf[DH / 16][4], dof[DH / 16][4];
  load_a_frags<DH>(qf, Qs + warp * 16 * LD, lane);
  load_a_frags<DH>(dof, dOs + warp * 16 * LD, lane);
  float L[2], Dl[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    int rloc = warp * 16 + g + r * 8;
    bool ok = rloc < len;
    L[r] = ok ? lse[(long long)(t0 + rloc) * H + h] : 0.f;
    Dl[r] = ok ? delta[(long long)(t0 + rloc) * H + h] : 0.f;
  }
  float acc[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
  const int nkv = (t0 - seq0) / 64 + 1;
  const int row0 = t0 + warp * 16 + g;
  for (int kt = 0; kt < nkv; ++kt) {
    const int kv0 = seq0 + kt * 64;
    const int kvlen = min(64, t0 + len - kv0);
    __syncthreads();
    load_tile<DH>(Ks, k, kv0, kvlen, H, h, tid, 128);
    load_tile<DH>(Vs, v, kv0, kvlen, H, h, tid, 128);
    __syncthreads();
    float s[8][4], dp[8][4];
    mma_a_bt<DH>(s, qf, Ks, lane);
    mma_a_bt<DH>(dp, dof, Vs, lane);
    const bool diag = (kt == nkv - 1);
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float p = exp2f(s[n][e] * scale_log2 - L[e >> 1]);
        if (diag) {
          int col = kv0 + n * 8 + 2 * tq + (e & 1);
          int row = row0 + (e >> 1) * 8;
          if (col > row) p = 0.f;
        }
        s[n][e] = p * (dp[n][e] - Dl[e >> 1]);          // dS
      }
    }
    mma_p_b<DH>(acc, s, Ks, lane);                       // dQ += dS K
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int rloc = warp * 16 + g + r * 8;
    if (rloc < len) {
      const long long tok = t0 + rloc;
#pragma unroll
      for (int n = 0; n < DH / 8; ++n)
        *(__nv_bfloat162*)(dq + (tok * H + h) * DH + n * 8 + 2 * tq) =
            __floats2bfloat162_rn(acc[n][2 * r] * scale, acc[n][2 * r + 1] * scale);
    }
  }
}

// dK, dV: one CTA per key tile, warps own 16 key rows, loop over the query tiles at or after it
template <int DH>
__global__ void __launch_bounds__(128)
attn_bwd_dkv_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                    const bf16* __restrict__ d_o, const float* __restrict__ lse, const float* __restrict__ delta,
                    const int* __restrict__ tile_start, const int* __restrict__ tile_len,
                    const int* __restrict__ tile_seq0, const int* __restrict__ tile_seq_end, int H, float scale_log2,
                    float scale, bf16* __restrict__ dk, bf16* __restrict__ dv) {
  constexpr int LD = DH + 8;
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* Ks = (bf16*)smem; bf16* Vs = Ks + 64 * LD; bf16* Qs = Vs + 64 * LD; bf16* dOs = Qs + 64 * LD;
  float* Ls = (float*)(dOs + 64 * LD); float* Ds = Ls + 64;
  const int tile = blockIdx.x, h = blockIdx.y;
  const int t0 = tile_start[tile], len = tile_len[tile], seq_end = tile_seq_end[tile];
  if (len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  load_tile<DH>(Ks, k, t0, len, H, h, tid, 128);
  load_tile<DH>(Vs, v, t0, len, H, h, tid, 128);
  __syncthreads();
  float dka[DH / 8][4], dva[DH / 8][4];
#pragma unroll
  for (int n = 0; n < DH / 8; ++n) {
    dka[n][0] = dka[n][1] = dka[n][2] = dka[n][3] = 0.f;
    dva[n][0] = dva[n][1] = dva[n][2] = dva[n][3] = 0.f;
  }
  const int krow0 = t0 + warp * 16 + g;                 // key token of this thread's first row
  for (int q0 = t0; q0 < seq_end; q0 += 64) {
    const int qlen = min(64, seq_end - q0);
    __syncthreads();
    load_tile<DH>(Qs, q, q0, qlen, H, h, tid, 128);
    load_tile<DH>(dOs, d_o, q0, qlen, H, h, tid, 128);
    if (tid < 64) {
      bool ok = tid < qlen;
      Ls[tid] = ok ? lse[(long long)(q0 + tid) * H + h] : INFINITY;      // p = 0 for rows past the document
      Ds[tid] = ok ? delta[(long long)(q0 + tid) * H + h] : 0.f;
    }
    __syncthreads();
    float st[8][4];
    {
      uint32_t kf[DH / 16][4];
      load_a_frags<DH>(kf, Ks + warp * 16 * LD, lane);
      mma_a_bt<DH>(st, kf, Qs, lane);                    // S^T (16 keys x 64 queries)
    }
    const bool diag = (q0 == t0);
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int qc = n * 8 + 2 * tq + (e & 1);
        float p = exp2f(st[n][e] * scale_log2 - Ls[qc]);
        if (diag) {
          int qtok = q0 + qc, ktok = krow0 + (e >> 1) * 8;
          if (ktok > qtok) p = 0.f;
        }
        st[n][e] = p;
      }
    }
    mma_p_b<DH>(dva, st, dOs, lane);                     // dV += P^T dO
    {
      float dpt[8][4];
      uint32_t vf[DH / 16][4];
      load_a_frags<DH>(vf, Vs + warp * 16 * LD, lane);
      mma_a_bt<DH>(dpt, vf, dOs, lane);                  // dP^T
#pragma unroll
      for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int qc = n * 8 + 2 * tq + (e & 1);
          st[n][e] *= (dpt[n][e] - Ds[qc]);              // dS^T
        }
      }
    }
    mma_p_b<DH>(dka, st, Qs, lane);                      // dK += dS^T Q
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int rloc = warp * 16 + g + r * 8;
    if (rloc < len) {
      const long long tok = t0 + rloc;
#pragma unroll
      for (int n = 0; n < DH / 8; ++n) {
        *(__nv_bfloat162*)(dk + (tok * H + h) * DH + n * 8 + 2 * tq) =
            __floats2bfloat162_rn(dka[n][2 * r] * scale, dka[n][2 * r + 1] * scale);
        *(__nv_bfloat162*)(dv + (tok * H + h) * DH + n * 8 + 2 * tq) =
            __floats2bfloat162_rn(dva[n][2 * r], dva[n][2 * r + 1]);
      }
    }
  }
}

// tile table: 64-row tiles that never straddle a document; also the document start / end of each tile
__global__ void attn_build_tiles_kernel(const int* __restrict__ cu, int N, int* __restrict__ tile_start,
                                        int* __restrict__ tile_len, int* __restrict__ tile_seq0,
                                        int* __restrict__ tile_seq_end, int nt_max) {
  __shared__ int total;
  extern __shared__ int first[];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int n = 0; n < N; ++n) { first[n] = acc; acc += (cu[n + 1] - cu[n] + 63) / 64; }
    total = acc;
  }
  __syncthreads();
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    int s0 = cu[n], e = cu[n + 1], c = first[n];
    for (int s = s0; s < e; s += 64, ++c)
      if (c < nt_max) { tile_start[c] = s; tile_len[c] = min(64, e - s); tile_seq0[c] = s0; tile_seq_end[c] = e; }
  }
  for (int c = total + threadIdx.x; c < nt_max; c += blockDim.x) { tile_start[c] = 0; tile_len[c] = 0; tile_seq0[c] = 0; tile_seq_end[c] = 0; }
}

}  // namespace hippo

using namespace hippo;
#define ST(s) ((cudaStream_t)(s))

extern "C" int hippo_attn_build_tiles(const int* cu, int N, int* ts, int* tl, int* t0, int* te, int nt_max, void* s) {
  attn_build_tiles_kernel<<<1, 256, (N + 1) * sizeof(int), ST(s)>>>(cu, N, ts, tl, t0, te, nt_max);
  return (int)cudaGetLastError();
}

template <int DH>
static int attn_fwd_launch(const void* q, const void* k, const void* v, const int* ts, const int* tl, const int* t0,
                           int NT, int H, float scale, void* o, float* lse, cudaStream_t s) {
  constexpr int SM = 3 * 64 * (DH + 8) * 2;
  auto kern = attn_fwd_kernel<DH>;
  static bool once = false;
  if (!once) { cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM); if (e) return (int)e; once = true; }
  kern<<<dim3(NT, H), 128, SM, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, ts, tl, t0, H,
                                    scale * 1.4426950408889634f, (bf16*)o, lse);
  return (int)cudaGetLastError();
}
extern "C" int hippo_attn_fwd(const void* q, const void* k, const void* v, const int* ts, const int* tl, const int* t0,
                              int NT, int H, int DH, float scale, void* o, float* lse, void* s) {
  if (NT == 0) return 0;
  if (DH == 128) return attn_fwd_launch<128>(q, k, v, ts, tl, t0, NT, H, scale, o, lse, ST(s));
  if (DH == 64) return attn_fwd_launch<64>(q, k, v, ts, tl, t0, NT, H, scale, o, lse, ST(s));
  return -1;
}

template <int DH>
static int attn_bwd_launch(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                           float* delta, const int* ts, const int* tl, const int* t0, const int* te, int NT, int H,
                           long long T, float scale, void* dq, void* dk, void* dv, cudaStream_t s) {
  constexpr int SMQ = 4 * 64 * (DH + 8) * 2;
  constexpr int SMK = 4 * 64 * (DH + 8) * 2 + 128 * 4;
  auto kq = attn_bwd_dq_kernel<DH>;
  auto kk = attn_bwd_dkv_kernel<DH>;
  static bool once = false;
  if (!once) {
    cudaError_t e = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, SMQ); if (e) return (int)e;
    e = cudaFuncSetAttribute(kk, cudaFuncAttributeMaxDynamicSharedMemorySize, SMK); if (e) return (int)e;
    once = true;
  }
  long long rows = T * H;
  attn_bwd_delta_kernel<DH><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const bf16*)o, (const bf16*)d_o, delta, rows);
  const float sl2 = scale * 1.4426950408889634f;
  kq<<<dim3(NT, H), 128, SMQ, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, (const bf16*)d_o, lse, delta, ts, tl,
                                   t0, H, sl2, scale, (bf16*)dq);
  kk<<<dim3(NT, H), 128, SMK, s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, (const bf16*)d_o, lse, delta, ts, tl,
                                   t0, te, H, sl2, scale, (bf16*)dk, (bf16*)dv);
  return (int)cudaGetLastError();
}
extern "C" int hippo_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                              const float* lse, float* delta, const int* ts, const int* tl, const int* t0, const int* te,
                              int NT, int H, int DH, long long T, float scale, void* dq, void* dk, void* dv, void* s) {
  if (NT == 0) return 0;
  if (DH == 128) return attn_bwd_launch<128>(q, k, v, o, d_o, lse, delta, ts, tl, t0, te, NT, H, T, scale, dq, dk, dv, ST(s));
  if (DH == 64) return attn_bwd_launch<64>(q, k, v, o, d_o, lse, delta, ts, tl, t0, te, NT, H, T, scale, dq, dk, dv, ST(s));
  return -1;
}
