// Block attention-residual mix (fwd/bwd), AdamW update, NVFP4 quantise / dequantise, cross-entropy
// row statistics and gradient, multi-tensor sum of squares. Memory-bound kernels, fp32 math.
// Reference behaviour: src/models/ops/attn_res_triton.py:108-521, param_offload/cpu_fused.py:532-583,
// src/models/ops/nvfp4_quant_triton.py:77-142, fla/modules/fused_linear_cross_entropy.py:43-358.
#include <cuda_runtime.h>
#include "sm100.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <stdint.h>

namespace hippo {
typedef __nv_bfloat16 bf16;
constexpr int AR_MAX = 16;
struct PtrList { const void* p[AR_MAX]; };
struct MutPtrList { void* p[AR_MAX]; };

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ void ld8(const bf16* p, float (&f)[8]) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(b[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ void st8(bf16* p, const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = v;
}

// ------------------------------------------------------------------------------------ AttnRes
// One block per token, D/8 threads (each owns 8 contiguous channels; a head spans GS = dh/8 lanes,
// GS a power of two <= 32). sources: N tensors [T, D]. Saves alpha [N,T,H] and rstd [N,T].
template <int NMAX>
__global__ void __launch_bounds__(512)
attnres_fwd_kernel(PtrList src, int N, const bf16* __restrict__ query, const bf16* __restrict__ w,
                   bf16* __restrict__ out, float* __restrict__ alpha, float* __restrict__ rstd,
                   long long T, int D, int H, float eps) {
  __shared__ float red[NMAX][32];
  const long long t = blockIdx.x;
  const int tid = threadIdx.x, c0 = tid * 8, dh = D / H, GS = dh / 8, h = c0 / dh;
  const int warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  float qw[8], fq[8], fw[8];
  ld8(query + c0, fq); ld8(w + c0, fw);
#pragma unroll
  for (int i = 0; i < 8; ++i) qw[i] = fq[i] * fw[i];
  float dot[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) {
    dot[n] = 0.f;
    if (n < N) {
      float v[8], ss = 0.f;
      ld8((const bf16*)src.p[n] + t * D + c0, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) { ss += v[i] * v[i]; dot[n] += v[i] * qw[i]; }
      for (int o = 1; o < GS; o <<= 1) dot[n] += __shfl_xor_sync(0xFFFFFFFFu, dot[n], o);
      float s = wsum(ss);
      if (lane == 0) red[n][warp] = s;
    }
  }
  __syncthreads();
  float mx = -INFINITY;
#pragma unroll
  for (int n = 0; n < NMAX; ++n) {
    if (n < N) {
      float s = 0.f;
      for (int k = 0; k < nw; ++k) s += red[n][k];
      float r = rsqrtf(s / D + eps);
      if (tid == 0) rstd[(long long)n * T + t] = r;
      dot[n] *= r;                                     // logit
      mx = fmaxf(mx, dot[n]);
    }
  }
  float den = 0.f;
#pragma unroll
  for (int n = 0; n < NMAX; ++n) if (n < N) { dot[n] = __expf(dot[n] - mx); den += dot[n]; }
  float o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
  for (int n = 0; n < NMAX; ++n) {
    if (n < N) {
      float a = dot[n] / den;
      if ((tid % GS) == 0) alpha[((long long)n * T + t) * H + h] = a;
      float v[8];
      ld8((const bf16*)src.p[n] + t * D + c0, v);      // second read hits L1/L2
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += a * v[i];
    }
  }
  st8(out + t * D + c0, o);
}

// grid-stride over tokens; dq/dw partials in registers, one atomicAdd per channel per block at the end
template <int NMAX>
__global__ void __launch_bounds__(512)
attnres_bwd_kernel(PtrList src, int N, const bf16* __restrict__ query, const bf16* __restrict__ w,
                   const bf16* __restrict__ out, const bf16* __restrict__ d_out,
                   const float* __restrict__ alpha, const float* __restrict__ rstd, MutPtrList dsrc,
                   float* __restrict__ dq, float* __restrict__ dw, long long T, int D, int H) {
  __shared__ float red[NMAX][32];
  const int tid = threadIdx.x, c0 = tid * 8, dh = D / H, GS = dh / 8, h = c0 / dh;
  const int warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  float fq[8], fw[8], dqa[8], dwa[8];
  ld8(query + c0, fq); ld8(w + c0, fw);
#pragma unroll
  for (int i = 0; i < 8; ++i) { dqa[i] = 0.f; dwa[i] = 0.f; }
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    float go[8], fo[8];
    ld8(d_out + t * D + c0, go); ld8(out + t * D + c0, fo);
    float dout_o = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) dout_o += go[i] * fo[i];
    for (int o = 1; o < GS; o <<= 1) dout_o += __shfl_xor_sync(0xFFFFFFFFu, dout_o, o);
    float ds[NMAX];
    __syncthreads();
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      ds[n] = 0.f;
      if (n < N) {
        float v[8];
        ld8((const bf16*)src.p[n] + t * D + c0, v);
        float dv = 0.f, dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) { dv += go[i] * v[i]; dot += v[i] * fq[i] * fw[i]; }
        for (int o = 1; o < GS; o <<= 1) { dv += __shfl_xor_sync(0xFFFFFFFFu, dv, o); dot += __shfl_xor_sync(0xFFFFFFFFu, dot, o); }
        float a = alpha[((long long)n * T + t) * H + h];
        float r = rstd[(long long)n * T + t];
        ds[n] = a * (dv - dout_o);
        // sum over heads of ds*logit: each head counted once (first lane of the head group)
        float contrib = ((tid % GS) == 0) ? ds[n] * dot * r : 0.f;
        contrib = wsum(contrib);
        if (lane == 0) red[n][warp] = contrib;
      }
    }
    __syncthreads();
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      if (n < N) {
        float sdl = 0.f;
        for (int k = 0; k < nw; ++k) sdl += red[n][k];
        float a = alpha[((long long)n * T + t) * H + h];
        float r = rstd[(long long)n * T + t];
        float v[8], dvn[8];
        ld8((const bf16*)src.p[n] + t * D + c0, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dvn[i] = a * go[i] + ds[n] * r * fq[i] * fw[i] - v[i] * r * r / D * sdl;
          dqa[i] += ds[n] * v[i] * r * fw[i];
          dwa[i] += ds[n] * fq[i] * v[i] * r;
        }
        st8((bf16*)dsrc.p[n] + t * D + c0, dvn);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) { atomicAdd(&dq[c0 + i], dqa[i]); atomicAdd(&dw[c0 + i], dwa[i]); }
}

// ------------------------------------------------------------------------------------ AdamW
__device__ __forceinline__ float ldf(const void* p, long long i, int is_bf16) {
  return is_bf16 ? __bfloat162float(((const bf16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ void stf(void* p, long long i, int is_bf16, float v) {
  if (is_bf16) ((bf16*)p)[i] = __float2bfloat16(v); else ((float*)p)[i] = v;
}
// standard AdamW: m,v EMA of g and g^2, both bias corrections, decoupled weight decay
__global__ void adamw_kernel(void* p, const void* g, void* m, void* v, long long n, int p_bf16, int g_bf16, int m_bf16,
                             int v_bf16, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                             float gscale) {
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float gv = ldf(g, i, g_bf16) * gscale;
  float mv = ldf(m, i, m_bf16) * b1 + (1.f - b1) * gv;
  float vv = ldf(v, i, v_bf16) * b2 + (1.f - b2) * gv * gv;
  stf(m, i, m_bf16, mv); stf(v, i, v_bf16, vv);
  float upd = (mv / bc1) / (sqrtf(vv / bc2) + eps);
  float pv = ldf(p, i, p_bf16);
  stf(p, i, p_bf16, pv * (1.f - lr * wd) - lr * upd);
}

// out[0] += sum x^2 (one atomicAdd per block)
__global__ void sumsq_kernel(const void* x, long long n, int is_bf16, float* out) {
  __shared__ float sh[32];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = ldf(x, i, is_bf16); s += v * v;
  }
  s = wsum(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    r = wsum(r);
    if (threadIdx.x == 0) atomicAdd(out, r);
  }
}

// Sum of squares of MANY tensors in one launch (the global gradient norm): one table entry per tensor segment,
// out[slot] += sum x^2. Blocks walk (entry, 2048-element piece) pairs; one atomicAdd per piece.
struct SumsqEntry { const void* ptr; long long n; int is_bf16; int slot; long long piece0; };
__global__ void sumsq_multi_kernel(const SumsqEntry* __restrict__ tab, int n_entries, long long n_pieces, float* out) {
  __shared__ float sh[32];
  for (long long pc = blockIdx.x; pc < n_pieces; pc += gridDim.x) {
    int lo = 0, hi = n_entries - 1;                       // last entry whose first piece is <= pc
    while (lo < hi) { int mid = (lo + hi + 1) >> 1; if (tab[mid].piece0 <= pc) lo = mid; else hi = mid - 1; }
    const SumsqEntry e = tab[lo];
    const long long i0 = (pc - e.piece0) * 2048;
    float s = 0.f;
    for (long long i = i0 + threadIdx.x; i < e.n && i < i0 + 2048; i += blockDim.x) { float v = ldf(e.ptr, i, e.is_bf16); s += v * v; }
    s = wsum(s);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
      float r = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
      r = wsum(r);
      if (threadIdx.x == 0) atomicAdd(out + e.slot, r);
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------ NVFP4
__global__ void absmax_kernel(const void* x, long long n, int is_bf16, float* out) {
  float m = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(ldf(x, i, is_bf16)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if ((threadIdx.x & 31) == 0) atomicMax((int*)out, __float_as_int(m));     // m >= 0: int order == float order
}
__global__ void nvfp4_global_scale_kernel(const float* amax, float* gs) {
  float a = *amax;
  *gs = a > 0.f ? a / (6.f * 448.f) : 1.f;
}
// one thread per 16-element block along K: e4m3 block scale = absmax/6/global, RN-even E2M1 codes,
// byte = even element | odd element << 4
__global__ void nvfp4_quant_kernel(const void* x, int is_bf16, long long nblocks, const float* gs_ptr,
                                   uint8_t* __restrict__ packed, uint8_t* __restrict__ scales) {
  long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const float gs = *gs_ptr;
  float f[16];
  if (is_bf16) { float a[8], c[8]; ld8((const bf16*)x + b * 16, a); ld8((const bf16*)x + b * 16 + 8, c);
#pragma unroll
    for (int i = 0; i < 8; ++i) { f[i] = a[i]; f[8 + i] = c[i]; } }
  else {
#pragma unroll
    for (int i = 0; i < 16; i += 4) { float4 t = *(const float4*)((const float*)x + b * 16 + i); f[i] = t.x; f[i + 1] = t.y; f[i + 2] = t.z; f[i + 3] = t.w; }
  }
  float bm = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) bm = fmaxf(bm, fabsf(f[i]));
  float sraw = fminf(bm / 6.f / gs, 448.f);
  __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(sraw, __NV_SATFINITE, __NV_E4M3);
  scales[b] = (uint8_t)s8;
  float sdec = __half2float(__half(__nv_cvt_fp8_to_halfraw(s8, __NV_E4M3))) * gs;
  float inv = sdec > 0.f ? 1.f / sdec : 1.f;
  uint2 outv;
  uint8_t* ob = (uint8_t*)&outv;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    // division (not reciprocal multiply) keeps ties identical to the torch oracle
    float lo = sdec > 0.f ? f[2 * i] / sdec : f[2 * i], hi = sdec > 0.f ? f[2 * i + 1] / sdec : f[2 * i + 1];
    (void)inv;
    ob[i] = (uint8_t)__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
  }
  *(uint2*)(packed + b * 8) = outv;
}
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                                     const float* gs_ptr, void* out, int out_bf16, long long nblocks) {
  long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const float lut[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  float s = __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)scales[b], __NV_E4M3))) * (*gs_ptr);
  uint2 pv = *(const uint2*)(packed + b * 8);
  const uint8_t* pb = (const uint8_t*)&pv;
  float f[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint8_t lo = pb[i] & 0xF, hi = pb[i] >> 4;
    f[2 * i] = ((lo & 8) ? -lut[lo & 7] : lut[lo & 7]) * s;
    f[2 * i + 1] = ((hi & 8) ? -lut[hi & 7] : lut[hi & 7]) * s;
  }
  if (out_bf16) {
    float a[8], c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = f[i]; c[i] = f[8 + i]; }
    st8((bf16*)out + b * 16, a); st8((bf16*)out + b * 16 + 8, c);
  } else {
#pragma unroll
    for (int i = 0; i < 16; i += 4) *(float4*)((float*)out + b * 16 + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
  }
}

// ------------------------------------------------------------------------------------ cross entropy rows
// per row of fp32 logits z[C, V]: max, sum exp(z - max), z[target] (0 when target < 0)
__global__ void ce_stats_kernel(const float* __restrict__ z, const long long* __restrict__ target, float* __restrict__ mx,
                                float* __restrict__ se, float* __restrict__ tz, int V) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const float* zr = z + row * V;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < V; c += blockDim.x) m = fmaxf(m, zr[c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = m;
  __syncthreads();
  m = sh[0];
  for (int k = 1; k < (blockDim.x >> 5); ++k) m = fmaxf(m, sh[k]);
  __syncthreads();
  float s = 0.f;
  for (int c = threadIdx.x; c < V; c += blockDim.x) s += __expf(zr[c] - m);
  s = wsum(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int k = 0; k < (blockDim.x >> 5); ++k) t += sh[k];
    mx[row] = m; se[row] = t;
    long long tg = target[row];
    tz[row] = (tg >= 0 && HIPPO_IN_BOUNDS(tg, V, 3)) ? zr[tg] : 0.f;     // targets < 0 are ignored rows
  }
}
// dz = (exp(z - lse) - onehot(target)) * w_row  as bf16, w_row = valid / n_valid
__global__ void ce_grad_kernel(const float* __restrict__ z, const float* __restrict__ lse,
                               const long long* __restrict__ target, const float* __restrict__ roww,
                               bf16* __restrict__ dz, int V) {
  const long long row = blockIdx.x;
  const float l = lse[row], w = roww[row];
  const long long tg = target[row];
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    float p = __expf(z[row * V + c] - l);
    if (c == tg) p -= 1.f;
    dz[row * V + c] = __float2bfloat16(p * w);
  }
}

}  // namespace hippo

using namespace hippo;
#define ST(s) ((cudaStream_t)(s))
#define RET() return (int)cudaGetLastError()

extern "C" int hippo_attnres_fwd(const void* const* srcs, int N, const void* query, const void* w, void* out, float* alpha,
                                 float* rstd, long long T, int D, int H, float eps, void* s) {
  if (N > AR_MAX || D % 8 || D / 8 > 512 || (D / H) % 8) return -1;
  int gs = (D / H) / 8;
  if (gs > 32 || (gs & (gs - 1))) return -2;
  PtrList pl; for (int i = 0; i < N; ++i) pl.p[i] = srcs[i];
  if (N <= 4) attnres_fwd_kernel<4><<<(unsigned)T, D / 8, 0, ST(s)>>>(pl, N, (const bf16*)query, (const bf16*)w, (bf16*)out, alpha, rstd, T, D, H, eps);
  else if (N <= 9) attnres_fwd_kernel<9><<<(unsigned)T, D / 8, 0, ST(s)>>>(pl, N, (const bf16*)query, (const bf16*)w, (bf16*)out, alpha, rstd, T, D, H, eps);
  else attnres_fwd_kernel<16><<<(unsigned)T, D / 8, 0, ST(s)>>>(pl, N, (const bf16*)query, (const bf16*)w, (bf16*)out, alpha, rstd, T, D, H, eps);
  RET();
}
extern "C" int hippo_attnres_bwd(const void* const* srcs, int N, const void* query, const void* w, const void* out,
                                 const void* d_out, const float* alpha, const float* rstd, void* const* dsrcs, float* dq,
                                 float* dw, long long T, int D, int H, void* s) {
  if (N > AR_MAX || D % 8 || D / 8 > 512) return -1;
  PtrList pl; MutPtrList dl;
  for (int i = 0; i < N; ++i) { pl.p[i] = srcs[i]; dl.p[i] = dsrcs[i]; }
  unsigned grid = (unsigned)(T < 592 ? T : 592);
  if (N <= 4) attnres_bwd_kernel<4><<<grid, D / 8, 0, ST(s)>>>(pl, N, (const bf16*)query, (const bf16*)w, (const bf16*)out, (const bf16*)d_out, alpha, rstd, dl, dq, dw, T, D, H);
  else if (N <= 9) attnres_bwd_kernel<9><<<grid, D / 8, 0, ST(s)>>>(pl, N, (const bf16*)query, (const bf16*)w, (const bf16*)out, (const bf16*)d_out, alpha, rstd, dl, dq, dw, T, D, H);
  else attnres_bwd_kernel<16><<<grid, D / 8, 0, ST(s)>>>(pl, N, (const bf16*)query, (const bf16*)w, (const bf16*)out, (const bf16*)d_out, alpha, rstd, dl, dq, dw, T, D, H);
  RET();
}
extern "C" int hippo_adamw(void* p, const void* g, void* m, void* v, long long n, int p_bf16, int g_bf16, int m_bf16,
                           int v_bf16, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                           float gscale, void* s) {
  adamw_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ST(s)>>>(p, g, m, v, n, p_bf16, g_bf16, m_bf16, v_bf16, lr, b1, b2, eps, wd, bc1, bc2, gscale);
  RET();
}
extern "C" int hippo_sumsq(const void* x, long long n, int is_bf16, float* out, void* s) {
  unsigned grid = (unsigned)((n + 256 * 8 - 1) / (256 * 8)); if (grid > 1184) grid = 1184; if (grid == 0) grid = 1;
  sumsq_kernel<<<grid, 256, 0, ST(s)>>>(x, n, is_bf16, out);
  RET();
}
// table: device array of n_entries SumsqEntry {ptr, n, is_bf16, slot, first piece index} (pieces of 2048 elements)
extern "C" int hippo_sumsq_multi(const void* table, int n_entries, long long n_pieces, float* out, void* s) {
  if (n_entries <= 0 || n_pieces <= 0) return 0;
  unsigned grid = (unsigned)(n_pieces < 2368 ? n_pieces : 2368);
  sumsq_multi_kernel<<<grid, 256, 0, ST(s)>>>((const SumsqEntry*)table, n_entries, n_pieces, out);
  RET();
}
// gs: device fp32[1]. compute_gs != 0: gs <- absmax(x)/(6*448) first (amax_scratch: device fp32[1])
extern "C" int hippo_nvfp4_quantize(const void* x, int is_bf16, long long rows, long long K, float* gs, int compute_gs,
                                    float* amax_scratch, void* packed, void* scales, void* s) {
  if (K % 16) return -1;
  long long n = rows * K, nb = n / 16;
  if (compute_gs) {
    cudaMemsetAsync(amax_scratch, 0, 4, ST(s));
    unsigned grid = (unsigned)((n + 2047) / 2048); if (grid > 1184) grid = 1184;
    absmax_kernel<<<grid, 256, 0, ST(s)>>>(x, n, is_bf16, amax_scratch);
    nvfp4_global_scale_kernel<<<1, 1, 0, ST(s)>>>(amax_scratch, gs);
  }
  nvfp4_quant_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, ST(s)>>>(x, is_bf16, nb, gs, (uint8_t*)packed, (uint8_t*)scales);
  RET();
}
// gs <- absmax(x)/(6*448) (1 when x is all zero). scratch, gs: device fp32[1]
extern "C" int hippo_nvfp4_tensor_scale(const void* x, long long n, int is_bf16, float* scratch, float* gs, void* s) {
  cudaMemsetAsync(scratch, 0, 4, ST(s));
  unsigned grid = (unsigned)((n + 2047) / 2048); if (grid > 1184) grid = 1184; if (grid == 0) grid = 1;
  absmax_kernel<<<grid, 256, 0, ST(s)>>>(x, n, is_bf16, scratch);
  nvfp4_global_scale_kernel<<<1, 1, 0, ST(s)>>>(scratch, gs);
  RET();
}
extern "C" int hippo_nvfp4_dequantize(const void* packed, const void* scales, const float* gs, void* out, int out_bf16,
                                      long long rows, long long K, void* s) {
  long long nb = rows * K / 16;
  nvfp4_dequant_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, ST(s)>>>((const uint8_t*)packed, (const uint8_t*)scales, gs, out, out_bf16, nb);
  RET();
}
extern "C" int hippo_ce_stats(const float* z, const long long* target, float* mx, float* se, float* tz, long long C, int V, void* s) {
  ce_stats_kernel<<<(unsigned)C, 512, 0, ST(s)>>>(z, target, mx, se, tz, V);
  RET();
}
extern "C" int hippo_ce_grad(const float* z, const float* lse, const long long* target, const float* roww, void* dz,
                             long long C, int V, void* s) {
  ce_grad_kernel<<<(unsigned)C, 512, 0, ST(s)>>>(z, lse, target, roww, (bf16*)dz, V);
  RET();
}

// ------------------------------------------------------------------------------------ Muon elementwise
namespace hippo {
// m <- beta*m + g*gscale ; u <- g*gscale + beta*m (nesterov) or m ; ssq += sum u^2.  8 elements per thread.
__global__ void muon_momentum_kernel(const void* g, int g_bf16, void* m, int m_bf16, bf16* __restrict__ u, long long n,
                                     float beta, float gscale, int nesterov, float* ssq) {
  __shared__ float sh[32];
  float acc = 0.f;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (long long)gridDim.x * blockDim.x * 8) {
    float gv[8], mv[8], uv[8];
    if (g_bf16) ld8((const bf16*)g + i, gv); else { float4 a = *(const float4*)((const float*)g + i), b = *(const float4*)((const float*)g + i + 4); gv[0]=a.x;gv[1]=a.y;gv[2]=a.z;gv[3]=a.w;gv[4]=b.x;gv[5]=b.y;gv[6]=b.z;gv[7]=b.w; }
    if (m_bf16) ld8((const bf16*)m + i, mv); else { float4 a = *(const float4*)((const float*)m + i), b = *(const float4*)((const float*)m + i + 4); mv[0]=a.x;mv[1]=a.y;mv[2]=a.z;mv[3]=a.w;mv[4]=b.x;mv[5]=b.y;mv[6]=b.z;mv[7]=b.w; }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float gg = gv[e] * gscale;
      mv[e] = beta * mv[e] + gg;
      uv[e] = nesterov ? gg + beta * mv[e] : mv[e];
      acc += uv[e] * uv[e];
    }
    if (m_bf16) st8((bf16*)m + i, mv); else { *(float4*)((float*)m + i) = make_float4(mv[0],mv[1],mv[2],mv[3]); *(float4*)((float*)m + i + 4) = make_float4(mv[4],mv[5],mv[6],mv[7]); }
    st8(u + i, uv);
  }
  acc = wsum(acc);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    r = wsum(r);
    if (threadIdx.x == 0) atomicAdd(ssq, r);
  }
}
// sum of squares of rows [r0, r1) of a row-major bf16 matrix (segment norms)
// x <- x / (sqrt(ssq) + eps)
__global__ void scale_inv_norm_kernel(bf16* __restrict__ x, long long n, const float* ssq, float eps) {
  const float s = 1.f / (sqrtf(*ssq) + eps);
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (long long)gridDim.x * blockDim.x * 8) {
    float v[8]; ld8(x + i, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= s;
    st8(x + i, v);
  }
}
// w <- w*wd - lr*o   (w bf16 or fp32, o bf16)
__global__ void axpby_update_kernel(void* w, int w_bf16, const bf16* __restrict__ o, long long n, float wd, float lr) {
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (long long)gridDim.x * blockDim.x * 8) {
    float ov[8], wv[8]; ld8(o + i, ov);
    if (w_bf16) ld8((const bf16*)w + i, wv); else { float4 a = *(const float4*)((const float*)w + i), b = *(const float4*)((const float*)w + i + 4); wv[0]=a.x;wv[1]=a.y;wv[2]=a.z;wv[3]=a.w;wv[4]=b.x;wv[5]=b.y;wv[6]=b.z;wv[7]=b.w; }
#pragma unroll
    for (int e = 0; e < 8; ++e) wv[e] = wv[e] * wd - lr * ov[e];
    if (w_bf16) st8((bf16*)w + i, wv); else { *(float4*)((float*)w + i) = make_float4(wv[0],wv[1],wv[2],wv[3]); *(float4*)((float*)w + i + 4) = make_float4(wv[4],wv[5],wv[6],wv[7]); }
  }
}
// NVFP4 weights without a master copy. One optimizer update of a tensor is three launches:
//   1. nvfp4_update_absmax_kernel   absmax of the UPDATED values w*wd - lr*o (nothing is written)
//   2. nvfp4_global_scale_kernel    tensor scale of the updated tensor, gs_new = absmax / (6 * 448)
//   3. nvfp4_apply_update_kernel    dequantise each 16-element block with the old tensor scale, update, re-quantise
//                                   against gs_new with a block scale rounded UP to e4m3 (no element exceeds 6 block
//                                   scales, so nothing saturates however far the weights have grown) and E2M1 codes
//                                   chosen by STOCHASTIC rounding.
// Round-to-nearest would drop every update smaller than half a code step (most Muon steps are), so a no-master weight
// would stop learning; with stochastic rounding the expected stored value equals the exact updated value.
// Random numbers: Philox4x32-10 keyed by (seed, 0) with the block index as counter: reproducible for a given seed,
// independent of the launch geometry.
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += 0x9E3779B9u; k.y += 0xBB67AE85u;
  }
  return c;
}
__device__ __forceinline__ void nvfp4_updated_block(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                                                    float gs, const bf16* __restrict__ o, long long b, float wd, float lr,
                                                    float (&f)[16], float& bm) {
  const float lut[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  float s = __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)scales[b], __NV_E4M3))) * gs;
  uint2 pv = *(const uint2*)(packed + b * 8);
  const uint8_t* pb = (const uint8_t*)&pv;
  float a[8], c[8];
  ld8(o + b * 16, a); ld8(o + b * 16 + 8, c);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint8_t lo = pb[i] & 0xF, hi = pb[i] >> 4;
    f[2 * i] = ((lo & 8) ? -lut[lo & 7] : lut[lo & 7]) * s;
    f[2 * i + 1] = ((hi & 8) ? -lut[hi & 7] : lut[hi & 7]) * s;
  }
  bm = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) { f[i] = f[i] * wd - lr * (i < 8 ? a[i] : c[i - 8]); bm = fmaxf(bm, fabsf(f[i])); }
}
__global__ void nvfp4_update_absmax_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                                           const float* gs_ptr, const bf16* __restrict__ o, long long nblocks, float wd,
                                           float lr, float* amax) {
  const float gs = *gs_ptr;
  float m = 0.f;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nblocks; b += (long long)gridDim.x * blockDim.x) {
    float f[16], bm;
    nvfp4_updated_block(packed, scales, gs, o, b, wd, lr, f, bm);
    m = fmaxf(m, bm);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
  if ((threadIdx.x & 31) == 0) atomicMax((int*)amax, __float_as_int(m));
}
// E2M1 code (magnitude index 0..7) of |x| <= 6 by stochastic rounding with u uniform in [0, 1)
__device__ __forceinline__ uint8_t e2m1_sr(float x, float u) {
  const float ax = fminf(fabsf(x), 6.f);
  // grid 0, .5, 1, 1.5, 2, 3, 4, 6: step .5 below 2, 1 below 4, 2 above
  float lo, step; int idx;
  if (ax < 2.f) { idx = (int)(ax * 2.f); lo = idx * .5f; step = .5f; }
  else if (ax < 4.f) { idx = 4 + (int)(ax - 2.f); lo = 2.f + (float)(idx - 4); step = 1.f; }
  else { idx = ax < 6.f ? 6 : 7; lo = idx == 6 ? 4.f : 6.f; step = 2.f; }
  if (idx < 7 && u < (ax - lo) / step) ++idx;
  return (uint8_t)(idx | (x < 0.f ? 8 : 0));
}
__global__ void nvfp4_apply_update_kernel(uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, const float* gs_old_ptr,
                                          const float* gs_new_ptr, const bf16* __restrict__ o, long long nblocks,
                                          long long block0, float wd, float lr, uint32_t seed, int stochastic) {
  long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nblocks) return;
  const float gs_new = *gs_new_ptr;
  float f[16], bm;
  nvfp4_updated_block(packed, scales, *gs_old_ptr, o, b, wd, lr, f, bm);
  // block scale rounded up to the next e4m3 value: absmax / scale <= 6, nothing clips
  const float sraw = fminf(bm / 6.f / gs_new, 448.f);
  __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(sraw, __NV_SATFINITE, __NV_E4M3);
  if (__half2float(__half(__nv_cvt_fp8_to_halfraw(s8, __NV_E4M3))) < sraw && s8 < 0x7E) ++s8;
  scales[b] = (uint8_t)s8;
  const float sdec = __half2float(__half(__nv_cvt_fp8_to_halfraw(s8, __NV_E4M3))) * gs_new;
  const float inv = sdec > 0.f ? 1.f / sdec : 0.f;
  uint2 outv; uint8_t* ob = (uint8_t*)&outv;
  if (stochastic) {
    const unsigned long long gb = (unsigned long long)(block0 + b);
    uint32_t r[8];
    uint4 r0 = philox4x32_10(make_uint4((uint32_t)gb, (uint32_t)(gb >> 32), 0u, 0u), make_uint2(seed, 0x5EEDu));
    uint4 r1 = philox4x32_10(make_uint4((uint32_t)gb, (uint32_t)(gb >> 32), 1u, 0u), make_uint2(seed, 0x5EEDu));
    r[0] = r0.x; r[1] = r0.y; r[2] = r0.z; r[3] = r0.w; r[4] = r1.x; r[5] = r1.y; r[6] = r1.z; r[7] = r1.w;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float u0 = (float)(r[i] & 0xFFFFu) * (1.f / 65536.f), u1 = (float)(r[i] >> 16) * (1.f / 65536.f);
      ob[i] = (uint8_t)(e2m1_sr(f[2 * i] * inv, u0) | (e2m1_sr(f[2 * i + 1] * inv, u1) << 4));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      ob[i] = (uint8_t)__nv_cvt_float2_to_fp4x2(make_float2(f[2 * i] * inv, f[2 * i + 1] * inv), __NV_E2M1, cudaRoundNearest);
  }
  *(uint2*)(packed + b * 8) = outv;
}
// vectorised AdamW for all-bf16 state (8 elements per thread)
__global__ void adamw_bf16_kernel(bf16* __restrict__ p, const bf16* __restrict__ g, bf16* __restrict__ m, bf16* __restrict__ v,
                                  long long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                                  float gscale) {
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += (long long)gridDim.x * blockDim.x * 8) {
    float pv[8], gv[8], mv[8], vv[8];
    ld8(p + i, pv); ld8(g + i, gv); ld8(m + i, mv); ld8(v + i, vv);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float gg = gv[e] * gscale;
      mv[e] = mv[e] * b1 + (1.f - b1) * gg;
      vv[e] = vv[e] * b2 + (1.f - b2) * gg * gg;
      pv[e] = pv[e] * (1.f - lr * wd) - lr * (mv[e] / bc1) / (sqrtf(vv[e] / bc2) + eps);
    }
    st8(p + i, pv); st8(m + i, mv); st8(v + i, vv);
  }
}
}  // namespace hippo

static unsigned grid8(long long n) { long long b = (n / 8 + 255) / 256; if (b > 148 * 16) b = 148 * 16; if (b < 1) b = 1; return (unsigned)b; }

extern "C" int hippo_muon_momentum(const void* g, int g_bf16, void* m, int m_bf16, void* u, long long n, float beta,
                                   float gscale, int nesterov, float* ssq, void* s) {
  if (n % 8) return -1;
  cudaMemsetAsync(ssq, 0, 4, ST(s));
  muon_momentum_kernel<<<grid8(n), 256, 0, ST(s)>>>(g, g_bf16, m, m_bf16, (bf16*)u, n, beta, gscale, nesterov, ssq);
  RET();
}
extern "C" int hippo_scale_inv_norm(void* x, long long n, const float* ssq, float eps, void* s) {
  if (n % 8) return -1;
  scale_inv_norm_kernel<<<grid8(n), 256, 0, ST(s)>>>((bf16*)x, n, ssq, eps);
  RET();
}
extern "C" int hippo_axpby_update(void* w, int w_bf16, const void* o, long long n, float wd, float lr, void* s) {
  if (n % 8) return -1;
  axpby_update_kernel<<<grid8(n), 256, 0, ST(s)>>>(w, w_bf16, (const bf16*)o, n, wd, lr);
  RET();
}
// Pass 1 of a no-master NVFP4 update: amax <- max(amax, absmax(w*wd - lr*o)) over rows of one segment (amax: device
// fp32[1], zeroed by the caller before the first segment of a tensor).
extern "C" int hippo_nvfp4_update_absmax(const void* packed, const void* scales, const float* gs, const void* o,
                                         long long rows, long long K, float wd, float lr, float* amax, void* s) {
  if (K % 16) return -1;
  long long nb = rows * K / 16;
  unsigned grid = (unsigned)((nb + 255) / 256); if (grid > 2368) grid = 2368; if (grid == 0) grid = 1;
  nvfp4_update_absmax_kernel<<<grid, 256, 0, ST(s)>>>((const uint8_t*)packed, (const uint8_t*)scales, gs, (const bf16*)o, nb, wd, lr, amax);
  RET();
}
// gs_new <- amax / (6 * 448) (1 for an all-zero tensor)
extern "C" int hippo_nvfp4_scale_from_absmax(const float* amax, float* gs_new, void* s) {
  nvfp4_global_scale_kernel<<<1, 1, 0, ST(s)>>>(amax, gs_new);
  RET();
}
// Pass 2: rows of one segment re-quantised against gs_new (gs_old == gs_new keeps the tensor scale). block0 = index of the
// segment's first 16-element block inside the tensor (the random stream is a function of (seed, global block index)).
extern "C" int hippo_nvfp4_apply_update(void* packed, void* scales, const float* gs_old, const float* gs_new, const void* o,
                                        long long rows, long long K, long long block0, float wd, float lr, unsigned seed,
                                        int stochastic, void* s) {
  if (K % 16) return -1;
  long long nb = rows * K / 16;
  nvfp4_apply_update_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, ST(s)>>>((uint8_t*)packed, (uint8_t*)scales, gs_old, gs_new,
                                                                            (const bf16*)o, nb, block0, wd, lr, seed, stochastic);
  RET();
}
extern "C" int hippo_adamw_bf16(void* p, const void* g, void* m, void* v, long long n, float lr, float b1, float b2,
                                float eps, float wd, float bc1, float bc2, float gscale, void* s) {
  if (n % 8) return -1;
  adamw_bf16_kernel<<<grid8(n), 256, 0, ST(s)>>>((bf16*)p, (const bf16*)g, (bf16*)m, (bf16*)v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
  RET();
}
