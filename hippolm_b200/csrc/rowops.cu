// Bandwidth-bound row kernels: RMSNorm, gated per-head RMSNorm, SwiGLU, KDA prologue
// (SiLU + L2 norm + beta sigmoid), KDA gate activation, RoPE. bf16 in/out, fp32 math, 16-byte
// vector accesses. Each forward has its backward here. They replace the reference's Triton kernels
// (fla/modules/layernorm.py:194-458, fused_norm_gate.py:35-330, l2norm.py:25-112, gate.py:143-417).
#include <cuda_runtime.h>
#include "sm100.cuh"
#include <atomic>
#include <cuda_bf16.h>
#include <stdint.h>

namespace hippo {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float r = (threadIdx.x < nw) ? sh[threadIdx.x] : 0.f;
  if (w == 0) { r = warp_sum(r); if (l == 0) sh[0] = r; }
  __syncthreads();
  return sh[0];
}
__device__ __forceinline__ void load8(const bf16* p, float (&f)[8]) {
  uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(b[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ void store8(bf16* p, const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = v;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------------------------ RMSNorm
// one block per row; D % 8 == 0
__global__ void rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                                   float* __restrict__ rstd, int D, float eps) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const bf16* xr = x + row * D;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) {
    float f[8]; load8(xr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = block_sum(ss, sh);
  float r = rsqrtf(ss / D + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  bf16* yr = y + row * D;
  for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) {
    float f[8], g[8]; load8(xr + c, f); load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * r * g[i];
    store8(yr + c, f);
  }
}

// s = x + res (stored, bf16), y = rmsnorm(s) * w: the residual add of a pre-norm layer fused into the norm that follows it
__global__ void add_rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, const bf16* __restrict__ w,
                                       bf16* __restrict__ sum, bf16* __restrict__ y, float* __restrict__ rstd, int D,
                                       float eps) {
  __shared__ float sh[32];
  const long long row = blockIdx.x;
  const bf16* xr = x + row * D; const bf16* rr = res + row * D;
  bf16* sr = sum + row * D;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) {
    float f[8], g[8]; load8(xr + c, f); load8(rr + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] + g[i]));   // the stored value is what is normalised
    store8(sr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = block_sum(ss, sh);
  float r = rsqrtf(ss / D + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  bf16* yr = y + row * D;
  for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) {     // each thread re-reads the pieces it wrote itself
    float f[8], g[8]; load8(sr + c, f); load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * r * g[i];
    store8(yr + c, f);
  }
}

// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)); partial dw[blockIdx.x, :] = sum over this block's rows of dy*xhat
// grid-stride over rows; each thread owns columns {threadIdx.x*8 + k*blockDim.x*8}; D <= blockDim.x*8*MAXV
template <int MAXV>
__global__ void rmsnorm_bwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ dy,
                                   const float* __restrict__ rstd, bf16* __restrict__ dx, float* __restrict__ dw_part,
                                   int T, int D, const bf16* __restrict__ dres = nullptr) {
  __shared__ float sh[32];
  float dwacc[MAXV][8];
#pragma unroll
  for (int v = 0; v < MAXV; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[v][i] = 0.f;
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const bf16* xr = x + row * D; const bf16* dyr = dy + row * D;
    float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      int c = threadIdx.x * 8 + v * blockDim.x * 8;
      if (c < D) {
        float fx[8], fd[8], fw[8]; load8(xr + c, fx); load8(dyr + c, fd); load8(w + c, fw);
#pragma unroll
        for (int i = 0; i < 8; ++i) { float xh = fx[i] * r; dot += fw[i] * fd[i] * xh; dwacc[v][i] += fd[i] * xh; }
      }
    }
    dot = block_sum(dot, sh) / D;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      int c = threadIdx.x * 8 + v * blockDim.x * 8;
      if (c < D) {
        float fx[8], fd[8], fw[8], o[8]; load8(xr + c, fx); load8(dyr + c, fd); load8(w + c, fw);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = r * (fw[i] * fd[i] - fx[i] * r * dot);
        if (dres) {                                       // gradient that reaches x through the residual path
          float fr[8]; load8(dres + row * D + c, fr);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += fr[i];
        }
        store8(dx + row * D + c, o);
      }
    }
  }
#pragma unroll
  for (int v = 0; v < MAXV; ++v) {
    int c = threadIdx.x * 8 + v * blockDim.x * 8;
    if (c < D) {
      float* dst = dw_part + (long long)blockIdx.x * D + c;
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[i] = dwacc[v][i];
    }
  }
}

__global__ void colsum_kernel(const float* __restrict__ part, float* __restrict__ out, int nparts, int D) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += part[(long long)p * D + c];
  out[c] = s;
}

// ------------------------------------------------------------------------------------ gated per-head RMSNorm
// rows = T*H of length V (V == 128 or 64: one warp per row, V/32 elements per lane, V % 32 == 0, V <= 256)
template <int VPL>
__global__ void gated_rmsnorm_fwd_kernel(const bf16* __restrict__ o, const bf16* __restrict__ gate,
                                         const bf16* __restrict__ w, bf16* __restrict__ y, float* __restrict__ rstd,
                                         long long rows, float eps) {
  const int V = VPL * 32;
  long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  int lane = threadIdx.x & 31;
  float f[VPL], g[VPL];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    f[i] = __bfloat162float(o[row * V + lane + 32 * i]);
    g[i] = __bfloat162float(gate[row * V + lane + 32 * i]);
    ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  float r = rsqrtf(ss / V + eps);
  if (lane == 0) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    float wv = __bfloat162float(w[lane + 32 * i]);
    y[row * V + lane + 32 * i] = __float2bfloat16(f[i] * r * wv * sigmoidf_(g[i]));
  }
}

template <int VPL>
__global__ void gated_rmsnorm_bwd_kernel(const bf16* __restrict__ o, const bf16* __restrict__ gate,
                                         const bf16* __restrict__ w, const bf16* __restrict__ dy,
                                         const float* __restrict__ rstd, bf16* __restrict__ d_o,
                                         bf16* __restrict__ dgate, float* __restrict__ dw, long long rows) {
  const int V = VPL * 32;
  __shared__ float shw[8][VPL * 32];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float dwacc[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) dwacc[i] = 0.f;
  for (long long row = (long long)blockIdx.x * nw + wid; row < rows; row += (long long)gridDim.x * nw) {
    float r = rstd[row];
    float n[VPL], dn[VPL];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      int c = lane + 32 * i;
      float ov = __bfloat162float(o[row * V + c]);
      float gv = __bfloat162float(gate[row * V + c]);
      float dyv = __bfloat162float(dy[row * V + c]);
      float wv = __bfloat162float(w[c]);
      float s = sigmoidf_(gv);
      n[i] = ov * r;
      dn[i] = dyv * wv * s;
      dot += dn[i] * n[i];
      dwacc[i] += dyv * n[i] * s;
      dgate[row * V + c] = __float2bfloat16(dyv * n[i] * wv * s * (1.f - s));
    }
    dot = warp_sum(dot) / V;
#pragma unroll
    for (int i = 0; i < VPL; ++i) d_o[row * V + lane + 32 * i] = __float2bfloat16(r * (dn[i] - n[i] * dot));
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) shw[wid][lane + 32 * i] = dwacc[i];
  __syncthreads();
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < nw; ++k) s += shw[k][c];
    atomicAdd(&dw[c], s);
  }
}

// ------------------------------------------------------------------------------------ SwiGLU
// gu: [T, 2I] (gate | up), a: [T, I]
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ a, long long T, int I) {
  long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  long long total = T * I;
  if (idx >= total) return;
  long long t = idx / I; int c = (int)(idx % I);
  float g[8], u[8], o[8];
  load8(gu + t * 2 * I + c, g); load8(gu + t * 2 * I + I + c, u);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = g[i] * sigmoidf_(g[i]) * u[i];
  store8(a + idx, o);
}
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ da, bf16* __restrict__ dgu,
                                  long long T, int I) {
  long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  long long total = T * I;
  if (idx >= total) return;
  long long t = idx / I; int c = (int)(idx % I);
  float g[8], u[8], d[8], dg[8], du[8];
  load8(gu + t * 2 * I + c, g); load8(gu + t * 2 * I + I + c, u); load8(da + idx, d);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float s = sigmoidf_(g[i]);
    dg[i] = d[i] * u[i] * s * (1.f + g[i] * (1.f - s));
    du[i] = d[i] * g[i] * s;
  }
  store8(dgu + t * 2 * I + c, dg); store8(dgu + t * 2 * I + I + c, du);
}

// ------------------------------------------------------------------------------------ KDA prologue
// proj row layout (stride ld): [q (H*K) | k (H*K) | v (H*V) | fg (2*Vd) | b (H) | pad].
// q,k <- l2norm(silu(.)) (q additionally * scale), v <- silu(.), beta <- sigmoid(b) * beta_mul.
// One warp per (token, head); K == V == 128 or 64 (KPL elements per lane).
template <int KPL>
__global__ void kda_prologue_fwd_kernel(const bf16* __restrict__ proj, long long ld, int H, int off_q, int off_k,
                                        int off_v, int off_b, bf16* __restrict__ q, bf16* __restrict__ k,
                                        bf16* __restrict__ v, float* __restrict__ beta, float* __restrict__ q_rstd,
                                        float* __restrict__ k_rstd, long long T, float scale, float beta_mul,
                                        int apply_silu) {
  const int K = KPL * 32;
  long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T * H) return;
  int lane = threadIdx.x & 31;
  long long t = row / H; int h = (int)(row % H);
  const bf16* pr = proj + t * ld;
  float fq[KPL], fk[KPL], sq = 0.f, sk = 0.f;
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    int c = h * K + lane + 32 * i;
    float a = __bfloat162float(pr[off_q + c]), b = __bfloat162float(pr[off_k + c]), cv = __bfloat162float(pr[off_v + c]);
    if (apply_silu) { a = a * sigmoidf_(a); b = b * sigmoidf_(b); cv = cv * sigmoidf_(cv); }
    fq[i] = a; fk[i] = b; sq += a * a; sk += b * b;
    v[row * K + lane + 32 * i] = __float2bfloat16(cv);
  }
  sq = warp_sum(sq); sk = warp_sum(sk);
  float rq = rsqrtf(sq + 1e-6f), rk = rsqrtf(sk + 1e-6f);
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    q[row * K + lane + 32 * i] = __float2bfloat16(fq[i] * rq * scale);
    k[row * K + lane + 32 * i] = __float2bfloat16(fk[i] * rk);
  }
  if (lane == 0) {
    q_rstd[row] = rq; k_rstd[row] = rk;
    beta[row] = sigmoidf_(__bfloat162float(pr[off_b + h])) * beta_mul;
  }
}

// backward into dproj columns q,k,v,b (fg columns and pad are written by the caller)
template <int KPL>
__global__ void kda_prologue_bwd_kernel(const bf16* __restrict__ proj, long long ld, int H, int off_q, int off_k,
                                        int off_v, int off_b, const bf16* __restrict__ dq, const bf16* __restrict__ dk,
                                        const bf16* __restrict__ dv, const float* __restrict__ dbeta,
                                        const float* __restrict__ q_rstd, const float* __restrict__ k_rstd,
                                        bf16* __restrict__ dproj, long long T, float scale, float beta_mul,
                                        int apply_silu) {
  const int K = KPL * 32;
  long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T * H) return;
  int lane = threadIdx.x & 31;
  long long t = row / H; int h = (int)(row % H);
  const bf16* pr = proj + t * ld;
  bf16* dp = dproj + t * ld;
  float rq = q_rstd[row], rk = k_rstd[row];
  float xq[KPL], xk[KPL], sq_[KPL], sk_[KPL], gq[KPL], gk[KPL], dotq = 0.f, dotk = 0.f;
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    int c = h * K + lane + 32 * i;
    float a = __bfloat162float(pr[off_q + c]), b = __bfloat162float(pr[off_k + c]);
    xq[i] = a; xk[i] = b;
    sq_[i] = apply_silu ? a * sigmoidf_(a) : a;
    sk_[i] = apply_silu ? b * sigmoidf_(b) : b;
    gq[i] = __bfloat162float(dq[row * K + lane + 32 * i]) * scale;        // grad wrt normalised (unscaled) q
    gk[i] = __bfloat162float(dk[row * K + lane + 32 * i]);
    dotq += gq[i] * sq_[i]; dotk += gk[i] * sk_[i];
  }
  dotq = warp_sum(dotq); dotk = warp_sum(dotk);
#pragma unroll
  for (int i = 0; i < KPL; ++i) {
    int c = h * K + lane + 32 * i;
    // y = s * r, r = (sum s^2 + eps)^-1/2 : ds = r*g - s * r^3 * <g, s>
    float dsq = rq * gq[i] - sq_[i] * rq * rq * rq * dotq;
    float dsk = rk * gk[i] - sk_[i] * rk * rk * rk * dotk;
    float cv = __bfloat162float(pr[off_v + c]);
    float dvv = __bfloat162float(dv[row * K + lane + 32 * i]);
    if (apply_silu) {
      float s1 = sigmoidf_(xq[i]); dsq *= s1 * (1.f + xq[i] * (1.f - s1));
      float s2 = sigmoidf_(xk[i]); dsk *= s2 * (1.f + xk[i] * (1.f - s2));
      float s3 = sigmoidf_(cv); dvv *= s3 * (1.f + cv * (1.f - s3));
    }
    dp[off_q + c] = __float2bfloat16(dsq);
    dp[off_k + c] = __float2bfloat16(dsk);
    dp[off_v + c] = __float2bfloat16(dvv);
  }
  if (lane == 0) {
    float s = sigmoidf_(__bfloat162float(pr[off_b + h]));
    dp[off_b + h] = __float2bfloat16(dbeta[row] * beta_mul * s * (1.f - s));
  }
}

// ------------------------------------------------------------------------------------ KDA gate
// g[t,h,c] = -exp(A[h]) * softplus(x + b[h,c])            (plain)
//          = lower * sigmoid(exp(A[h]) * (x + b[h,c]))     (safe)
__global__ void kda_gate_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ A, const float* __restrict__ b,
                                    float* __restrict__ g, long long T, int H, int K, int safe, float lower) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * H * K) return;
  int hk = (int)(idx % ((long long)H * K)); int h = hk / K;
  float a = __expf(A[h]);
  float z = __bfloat162float(x[idx]) + (b ? b[hk] : 0.f);
  float out;
  if (safe) out = lower * sigmoidf_(a * z);
  else out = -a * (z > 20.f ? z : log1pf(__expf(z)));
  g[idx] = out;
}
// dx[t,h,c]; dA[h] += sum dg*dg/dA ; db[h,c] += sum dg*dg/dz.  grid: (HK/blockDim, T-splits)
__global__ void kda_gate_bwd_kernel(const bf16* __restrict__ x, const float* __restrict__ A, const float* __restrict__ b,
                                    const float* __restrict__ dg, bf16* __restrict__ dx, float* __restrict__ dA,
                                    float* __restrict__ db, long long T, int H, int K, int safe, float lower) {
  int hk = blockIdx.x * blockDim.x + threadIdx.x;
  int HK = H * K;
  if (hk >= HK) return;
  int h = hk / K;
  float a = __expf(A[h]);
  float bb = b ? b[hk] : 0.f;
  float accA = 0.f, accB = 0.f;
  for (long long t = blockIdx.y; t < T; t += gridDim.y) {
    long long idx = t * HK + hk;
    float z = __bfloat162float(x[idx]) + bb;
    float d = dg[idx];
    float dz, da;
    if (safe) {
      float s = sigmoidf_(a * z);
      float ds = lower * s * (1.f - s);
      dz = d * ds * a; da = d * ds * z * a;          // d/dA_log = d/da * a
    } else {
      float sp = z > 20.f ? z : log1pf(__expf(z));
      dz = d * (-a) * sigmoidf_(z); da = d * (-a) * sp;
    }
    dx[idx] = __float2bfloat16(dz);
    accA += da; accB += dz;
  }
  if (db) atomicAdd(&db[hk], accB);
  // reduce accA over the K channels of head h: K is a multiple of 32 so a warp covers one head
  accA = warp_sum(accA);
  if ((threadIdx.x & 31) == 0) atomicAdd(&dA[h], accA);
}

// ------------------------------------------------------------------------------------ RoPE (rotate-half)
// x: [T, H, dh] rotated in place into out; sign = +1 forward, -1 backward (inverse rotation)
__global__ void rope_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, const int* __restrict__ pos,
                            long long T, int H, int dh, float theta_log2, float sign) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  int half = dh / 2;
  if (idx >= T * H * half) return;
  int i = (int)(idx % half);
  long long th = idx / half;
  long long t = th / H;
  float inv = exp2f(-theta_log2 * (2.f * i / dh));
  float ang = pos[t] * inv;
  float s, c; sincosf(ang, &s, &c); s *= sign;
  float x1 = __bfloat162float(x[th * dh + i]), x2 = __bfloat162float(x[th * dh + half + i]);
  out[th * dh + i] = __float2bfloat16(x1 * c - x2 * s);
  out[th * dh + half + i] = __float2bfloat16(x2 * c + x1 * s);
}

// ------------------------------------------------------------------------------------ misc elementwise
__global__ void silu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long long n) {
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  float f[8]; load8(x + i, f);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = f[j] * sigmoidf_(f[j]);
  store8(y + i, f);
}

}  // namespace hippo

using namespace hippo;
#define ST(s) ((cudaStream_t)(s))
#define RET() return (int)cudaGetLastError()

extern "C" int hippo_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long T, int D, float eps, void* s) {
  if (D % 8) return -1;
  int th = D >= 2048 ? 256 : 128;
  rmsnorm_fwd_kernel<<<(unsigned)T, th, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (bf16*)y, rstd, D, eps);
  RET();
}
extern "C" int hippo_add_rmsnorm_fwd(const void* x, const void* res, const void* w, void* sum, void* y, float* rstd,
                                     long long T, int D, float eps, void* s) {
  if (D % 8) return -1;
  int th = D >= 2048 ? 256 : 128;
  add_rmsnorm_fwd_kernel<<<(unsigned)T, th, 0, ST(s)>>>((const bf16*)x, (const bf16*)res, (const bf16*)w, (bf16*)sum, (bf16*)y, rstd, D, eps);
  RET();
}
// RMSNorm backward plus the gradient that reaches the normalised tensor through the residual path: dx = dres + norm'(dy)
extern "C" int hippo_rmsnorm_bwd_res(const void* x, const void* w, const void* dy, const void* dres, const float* rstd,
                                     void* dx, float* dw_part, float* dw, long long T, int D, int nblocks, void* s) {
  if (D % 8 || D > 256 * 8 * 4) return -1;
  int maxv = (D + 2047) / 2048;
  if (maxv <= 1) rmsnorm_bwd_kernel<1><<<nblocks, 256, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, dw_part, (int)T, D, (const bf16*)dres);
  else if (maxv == 2) rmsnorm_bwd_kernel<2><<<nblocks, 256, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, dw_part, (int)T, D, (const bf16*)dres);
  else rmsnorm_bwd_kernel<4><<<nblocks, 256, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, dw_part, (int)T, D, (const bf16*)dres);
  colsum_kernel<<<(D + 255) / 256, 256, 0, ST(s)>>>(dw_part, dw, nblocks, D);
  RET();
}
// dw_part: [nblocks, D] fp32 scratch; dw: [D] fp32 out. returns nblocks used via *nblocks_io (in: capacity)
extern "C" int hippo_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                                 float* dw_part, float* dw, long long T, int D, int nblocks, void* s) {
  if (D % 8 || D > 256 * 8 * 4) return -1;
  int maxv = (D + 2047) / 2048;
  if (maxv <= 1) rmsnorm_bwd_kernel<1><<<nblocks, 256, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, dw_part, (int)T, D);
  else if (maxv == 2) rmsnorm_bwd_kernel<2><<<nblocks, 256, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, dw_part, (int)T, D);
  else rmsnorm_bwd_kernel<4><<<nblocks, 256, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, dw_part, (int)T, D);
  colsum_kernel<<<(D + 255) / 256, 256, 0, ST(s)>>>(dw_part, dw, nblocks, D);
  RET();
}
extern "C" int hippo_gated_rmsnorm_fwd(const void* o, const void* gate, const void* w, void* y, float* rstd,
                                       long long rows, int V, float eps, void* s) {
  unsigned blocks = (unsigned)((rows + 7) / 8);
  if (V == 128) gated_rmsnorm_fwd_kernel<4><<<blocks, 256, 0, ST(s)>>>((const bf16*)o, (const bf16*)gate, (const bf16*)w, (bf16*)y, rstd, rows, eps);
  else if (V == 64) gated_rmsnorm_fwd_kernel<2><<<blocks, 256, 0, ST(s)>>>((const bf16*)o, (const bf16*)gate, (const bf16*)w, (bf16*)y, rstd, rows, eps);
  else if (V == 32) gated_rmsnorm_fwd_kernel<1><<<blocks, 256, 0, ST(s)>>>((const bf16*)o, (const bf16*)gate, (const bf16*)w, (bf16*)y, rstd, rows, eps);
  else return -1;
  RET();
}
extern "C" int hippo_gated_rmsnorm_bwd(const void* o, const void* gate, const void* w, const void* dy, const float* rstd,
                                       void* d_o, void* dgate, float* dw, long long rows, int V, void* s) {
  unsigned blocks = 148 * 4;
  if (V == 128) gated_rmsnorm_bwd_kernel<4><<<blocks, 256, 0, ST(s)>>>((const bf16*)o, (const bf16*)gate, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)d_o, (bf16*)dgate, dw, rows);
  else if (V == 64) gated_rmsnorm_bwd_kernel<2><<<blocks, 256, 0, ST(s)>>>((const bf16*)o, (const bf16*)gate, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)d_o, (bf16*)dgate, dw, rows);
  else if (V == 32) gated_rmsnorm_bwd_kernel<1><<<blocks, 256, 0, ST(s)>>>((const bf16*)o, (const bf16*)gate, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)d_o, (bf16*)dgate, dw, rows);
  else return -1;
  RET();
}
extern "C" int hippo_swiglu_fwd(const void* gu, void* a, long long T, int I, void* s) {
  if (I % 8) return -1;
  long long n = T * I / 8;
  swiglu_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ST(s)>>>((const bf16*)gu, (bf16*)a, T, I);
  RET();
}
extern "C" int hippo_swiglu_bwd(const void* gu, const void* da, void* dgu, long long T, int I, void* s) {
  if (I % 8) return -1;
  long long n = T * I / 8;
  swiglu_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ST(s)>>>((const bf16*)gu, (const bf16*)da, (bf16*)dgu, T, I);
  RET();
}
extern "C" int hippo_kda_prologue_fwd(const void* proj, long long ld, int H, int K, int off_q, int off_k, int off_v,
                                      int off_b, void* q, void* k, void* v, float* beta, float* q_rstd, float* k_rstd,
                                      long long T, float scale, float beta_mul, int apply_silu, void* s) {
  unsigned blocks = (unsigned)((T * H + 7) / 8);
  if (K == 128) kda_prologue_fwd_kernel<4><<<blocks, 256, 0, ST(s)>>>((const bf16*)proj, ld, H, off_q, off_k, off_v, off_b, (bf16*)q, (bf16*)k, (bf16*)v, beta, q_rstd, k_rstd, T, scale, beta_mul, apply_silu);
  else if (K == 64) kda_prologue_fwd_kernel<2><<<blocks, 256, 0, ST(s)>>>((const bf16*)proj, ld, H, off_q, off_k, off_v, off_b, (bf16*)q, (bf16*)k, (bf16*)v, beta, q_rstd, k_rstd, T, scale, beta_mul, apply_silu);
  else return -1;
  RET();
}
extern "C" int hippo_kda_prologue_bwd(const void* proj, long long ld, int H, int K, int off_q, int off_k, int off_v,
                                      int off_b, const void* dq, const void* dk, const void* dv, const float* dbeta,
                                      const float* q_rstd, const float* k_rstd, void* dproj, long long T, float scale,
                                      float beta_mul, int apply_silu, void* s) {
  unsigned blocks = (unsigned)((T * H + 7) / 8);
  if (K == 128) kda_prologue_bwd_kernel<4><<<blocks, 256, 0, ST(s)>>>((const bf16*)proj, ld, H, off_q, off_k, off_v, off_b, (const bf16*)dq, (const bf16*)dk, (const bf16*)dv, dbeta, q_rstd, k_rstd, (bf16*)dproj, T, scale, beta_mul, apply_silu);
  else if (K == 64) kda_prologue_bwd_kernel<2><<<blocks, 256, 0, ST(s)>>>((const bf16*)proj, ld, H, off_q, off_k, off_v, off_b, (const bf16*)dq, (const bf16*)dk, (const bf16*)dv, dbeta, q_rstd, k_rstd, (bf16*)dproj, T, scale, beta_mul, apply_silu);
  else return -1;
  RET();
}
extern "C" int hippo_kda_gate_fwd(const void* x, const float* A, const float* b, float* g, long long T, int H, int K,
                                  int safe, float lower, void* s) {
  long long n = T * H * K;
  kda_gate_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ST(s)>>>((const bf16*)x, A, b, g, T, H, K, safe, lower);
  RET();
}
extern "C" int hippo_kda_gate_bwd(const void* x, const float* A, const float* b, const float* dg, void* dx, float* dA,
                                  float* db, long long T, int H, int K, int safe, float lower, void* s) {
  if (K % 32) return -1;
  dim3 grid((H * K + 127) / 128, (unsigned)(T < 256 ? T : 256));
  kda_gate_bwd_kernel<<<grid, 128, 0, ST(s)>>>((const bf16*)x, A, b, dg, (bf16*)dx, dA, db, T, H, K, safe, lower);
  RET();
}
extern "C" int hippo_rope(const void* x, void* out, const int* pos, long long T, int H, int dh, float theta, float sign, void* s) {
  long long n = T * H * (dh / 2);
  rope_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ST(s)>>>((const bf16*)x, (bf16*)out, pos, T, H, dh, log2f(theta), sign);
  RET();
}
extern "C" int hippo_silu_fwd(const void* x, void* y, long long n, void* s) {
  if (n % 8) return -1;
  silu_fwd_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, ST(s)>>>((const bf16*)x, (bf16*)y, n);
  RET();
}

// ---------------------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate device memory (declared in no_alloc.h).
// The per-block partial sums of dw, which hippo_rmsnorm_bwd takes as a caller-allocated buffer, live
// here in a fixed array inside the library image. Each GPU that loads the library carries its own copy
// of the array until the process exits.
namespace hippo {
constexpr int kNoAllocBlocks = 148;                    // one block per SM of a B200
constexpr int kNoAllocMaxD = 8192;                     // widest row the entry point accepts
static __device__ __align__(256) float g_noalloc_dw_part[kNoAllocBlocks * kNoAllocMaxD];   // 4.6 MiB
constexpr int kNoAllocMaxDevices = 64;
// device address of the array, per device; host threads may race to fill an entry, but they all store the same value,
// and the atomic keeps the store and the later loads well-defined
static std::atomic<float*> g_noalloc_ptr[kNoAllocMaxDevices];
}  // namespace hippo

extern "C" int hippo_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                                         float* dw, long long T, int D, void* s) {
  using namespace hippo;
  if (T <= 0 || D <= 0 || D % 8 != 0 || D > kNoAllocMaxD) return -22;      // wider than the built-in scratch
  if (T > 0x7fffffffLL) return -24;                                        // the kernels index rows with 32-bit ints
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoAllocMaxDevices) return -23;
  float* part = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (part == nullptr) {
    // First call on this device: ask the runtime where this device's copy of the array lives. In host code
    // the array's name is only a handle; a kernel must be given the address obtained here.
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_dw_part);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_ptr[dev].store(p, std::memory_order_release);
    part = p;
  }
  const int nblocks = (int)(T < kNoAllocBlocks ? T : kNoAllocBlocks);
  const int maxv = (D + 2047) / 2048;
  // every block writes all D entries of its own row of `part`, so nothing has to be cleared between calls
  if (maxv <= 1) rmsnorm_bwd_kernel<1><<<nblocks, 256, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, part, (int)T, D);
  else if (maxv == 2) rmsnorm_bwd_kernel<2><<<nblocks, 256, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, part, (int)T, D);
  else rmsnorm_bwd_kernel<4><<<nblocks, 256, 0, ST(s)>>>((const bf16*)x, (const bf16*)w, (const bf16*)dy, rstd, (bf16*)dx, part, (int)T, D);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;                                     // do not sum partials that were never written
  colsum_kernel<<<(D + 255) / 256, 256, 0, ST(s)>>>(part, dw, nblocks, D);
  RET();
}

// ---------------------------------------------------------------------------------------------------
// Depthwise causal short convolution (width W <= 8) + SiLU over a packed token stream, with the taps
// reset at document starts (pos_in_doc[t] = position of token t inside its document).
//   y[t, d] = silu( sum_w weight[d, w] * x[t - (W-1) + w, d]  (taps with t - (W-1) + w before the doc start are 0) )
// Replaces fla/modules/conv/triton/kernels.py:36-153 (causal_conv1d fwd/bwd) for the use_short_conv option.
namespace hippo {
__global__ void short_conv_fwd_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w,
                                      const int* __restrict__ pos, bf16* __restrict__ y, long long T, int D, int W) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * D) return;
  long long t = idx / D; int d = (int)(idx % D);
  int p = pos[t];
  float acc = 0.f;
  for (int wi = 0; wi < W; ++wi) {
    int shift = W - 1 - wi;
    if (p >= shift) acc += __bfloat162float(w[d * W + wi]) * __bfloat162float(x[(t - shift) * ldx + d]);
  }
  y[idx] = __float2bfloat16(acc * sigmoidf_(acc));
}
// dx[t, d] = sum_w weight[d, w] * dpre[t + (W-1) - w, d] for targets inside the same document;
// dw[d, w] += sum_t dpre[t, d] * x[t - (W-1) + w, d].  dpre = dy * silu'(pre), pre recomputed.
__global__ void short_conv_bwd_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w,
                                      const int* __restrict__ pos, const bf16* __restrict__ dy, bf16* __restrict__ dx,
                                      long long lddx, float* __restrict__ dw, long long T, int D, int W) {
  // one thread per channel d, grid-stride over token ranges (blockIdx.y); dpre of the last W-1 tokens is recomputed
  int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float wv[8], dwacc[8];
  for (int i = 0; i < W; ++i) { wv[i] = __bfloat162float(w[d * W + i]); dwacc[i] = 0.f; }
  const long long per = (T + gridDim.y - 1) / gridDim.y;
  const long long t_lo = (long long)blockIdx.y * per, t_hi = t_lo + per < T ? t_lo + per : T;
  auto dpre_at = [&](long long t) -> float {
    int p = pos[t];
    float pre = 0.f;
    for (int wi = 0; wi < W; ++wi) { int sh = W - 1 - wi; if (p >= sh) pre += wv[wi] * __bfloat162float(x[(t - sh) * ldx + d]); }
    float s = sigmoidf_(pre);
    return __bfloat162float(dy[t * D + d]) * s * (1.f + pre * (1.f - s));
  };
  for (long long t = t_lo; t < t_hi; ++t) {
    // gradient wrt x[t]: contributions of outputs t .. t+W-1 that lie in the same document
    float g = 0.f;
    for (int sh = 0; sh < W; ++sh) {
      long long to = t + sh;
      if (to < T && pos[to] >= sh) g += wv[W - 1 - sh] * dpre_at(to);
    }
    dx[t * lddx + d] = __float2bfloat16(g);
    // weight gradient from output t
    float dp = dpre_at(t);
    int p = pos[t];
    for (int wi = 0; wi < W; ++wi) { int sh = W - 1 - wi; if (p >= sh) dwacc[wi] += dp * __bfloat162float(x[(t - sh) * ldx + d]); }
  }
  for (int i = 0; i < W; ++i) atomicAdd(&dw[d * W + i], dwacc[i]);
}

// Vectorised variants (D % 8 == 0, 16-byte aligned rows): a thread owns 8 channels and a run of `tt` tokens and slides
// a W-row window over them in registers, so every x / dy element is read once and every y / dx element written once
// with 16-byte accesses (the scalar kernels above re-read each x element W (forward) or ~W*W (backward) times through
// the cache with 2-byte accesses). A block is 32 channel groups x 8 token runs; the weight-gradient partial sums of the
// 8 runs are added in shared memory before one atomicAdd per (channel, tap) and block.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
  for (int e = 0; e < 4; ++e) { const float2 t = __bfloat1622float2(h[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = (__nv_bfloat162*)&v;
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
  return v;
}

template <int W>
__global__ void __launch_bounds__(256)
short_conv_fwd_vec_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w,
                          const int* __restrict__ pos, bf16* __restrict__ y, long long T, int D, int tt) {
  const int cg = blockIdx.x * 32 + (threadIdx.x & 31);
  const long long t_lo = ((long long)blockIdx.y * 8 + (threadIdx.x >> 5)) * tt;
  if (cg * 8 >= D || t_lo >= T) return;
  const long long t_hi = t_lo + tt < T ? t_lo + tt : T;
  float wv[W][8], win[W][8];
#pragma unroll
  for (int c = 0; c < 8; ++c)
#pragma unroll
    for (int wi = 0; wi < W; ++wi) { wv[wi][c] = __bfloat162float(w[(cg * 8 + c) * W + wi]); win[wi][c] = 0.f; }
  for (long long t = t_lo - (W - 1); t < t_hi; ++t) {
#pragma unroll
    for (int wi = 0; wi + 1 < W; ++wi)
#pragma unroll
      for (int c = 0; c < 8; ++c) win[wi][c] = win[wi + 1][c];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t >= 0) v = *(const uint4*)(x + t * ldx + cg * 8);
    unpack8(v, win[W - 1]);
    if (t < t_lo) continue;
    int p = pos[t];
    if (!HIPPO_IN_BOUNDS(p, t + 1, 5)) p = 0;                // a position cannot exceed the token index
    float o[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float acc = 0.f;
#pragma unroll
      for (int wi = 0; wi < W; ++wi) if (p >= W - 1 - wi) acc += wv[wi][c] * win[wi][c];
      o[c] = acc * sigmoidf_(acc);
    }
    *(uint4*)(y + t * D + cg * 8) = pack8(o);
  }
}

template <int W>
__global__ void __launch_bounds__(256)
short_conv_bwd_vec_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w,
                          const int* __restrict__ pos, const bf16* __restrict__ dy, bf16* __restrict__ dx,
                          long long lddx, float* __restrict__ dw, long long T, int D, int tt) {
  __shared__ float red[8][W * 8][33];                       // [token run][tap, channel][channel group]
  const int lane = threadIdx.x & 31, run = threadIdx.x >> 5;
  const int cg = blockIdx.x * 32 + lane;
  const long long t_lo = ((long long)blockIdx.y * 8 + run) * tt;
  const bool active = cg * 8 < D && t_lo < T;
  float dwacc[W][8];
#pragma unroll
  for (int wi = 0; wi < W; ++wi)
#pragma unroll
    for (int c = 0; c < 8; ++c) dwacc[wi][c] = 0.f;
  if (active) {
    const long long t_hi = t_lo + tt < T ? t_lo + tt : T;
    float wv[W][8], xw[W][8], dpw[W][8];
    int pw[W];
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int wi = 0; wi < W; ++wi) {
        wv[wi][c] = __bfloat162float(w[(cg * 8 + c) * W + wi]); xw[wi][c] = 0.f; dpw[wi][c] = 0.f;
      }
#pragma unroll
    for (int wi = 0; wi < W; ++wi) pw[wi] = 0;
    // window index i holds token t - (W-1) + i; dx of token t - (W-1) is complete once dpre[t] is known
    for (long long t = t_lo - (W - 1); t < t_hi + (W - 1); ++t) {
#pragma unroll
      for (int wi = 0; wi + 1 < W; ++wi) {
        pw[wi] = pw[wi + 1];
#pragma unroll
        for (int c = 0; c < 8; ++c) { xw[wi][c] = xw[wi + 1][c]; dpw[wi][c] = dpw[wi + 1][c]; }
      }
      uint4 v = make_uint4(0, 0, 0, 0);
      if (t >= 0 && t < T) v = *(const uint4*)(x + t * ldx + cg * 8);
      unpack8(v, xw[W - 1]);
      pw[W - 1] = 0;
#pragma unroll
      for (int c = 0; c < 8; ++c) dpw[W - 1][c] = 0.f;
      if (t >= t_lo && t < T) {
        const int p = pos[t];
        pw[W - 1] = p;
        float g[8];
        unpack8(*(const uint4*)(dy + t * D + cg * 8), g);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float pre = 0.f;
#pragma unroll
          for (int wi = 0; wi < W; ++wi) if (p >= W - 1 - wi) pre += wv[wi][c] * xw[wi][c];
          const float sg = sigmoidf_(pre);
          const float dp = g[c] * sg * (1.f + pre * (1.f - sg));
          dpw[W - 1][c] = dp;
          if (t < t_hi) {                                    // tokens past the run belong to the next run's weight gradient
#pragma unroll
            for (int wi = 0; wi < W; ++wi) if (p >= W - 1 - wi) dwacc[wi][c] += dp * xw[wi][c];
          }
        }
      }
      const long long td = t - (W - 1);
      if (td >= t_lo && td < t_hi) {
        float o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float acc = 0.f;
#pragma unroll
          for (int sh = 0; sh < W; ++sh) if (pw[sh] >= sh) acc += wv[W - 1 - sh][c] * dpw[sh][c];
          o[c] = acc;
        }
        *(uint4*)(dx + td * lddx + cg * 8) = pack8(o);
      }
    }
  }
#pragma unroll
  for (int wi = 0; wi < W; ++wi)
#pragma unroll
    for (int c = 0; c < 8; ++c) red[run][wi * 8 + c][lane] = dwacc[wi][c];
  __syncthreads();
  for (int i = threadIdx.x; i < W * 8 * 32; i += 256) {
    const int e = i >> 5, l = i & 31;                        // e = tap * 8 + channel
    const int d = (blockIdx.x * 32 + l) * 8 + (e & 7);
    if (d >= D) continue;
    float sum = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) sum += red[r][e][l];
    atomicAdd(&dw[d * W + (e >> 3)], sum);
  }
}
}  // namespace hippo

extern "C" int hippo_short_conv_fwd(const void* x, long long ldx, const void* w, const int* pos, void* y, long long T,
                                    int D, int W, void* s) {
  if (W > 8) return -1;
  if (T <= 0 || D <= 0) return 0;
  if (W == 4 && D % 8 == 0 && ldx % 8 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)y & 15)) {
    const int tt = 32;
    dim3 grid((D / 8 + 31) / 32, (unsigned)((T + 8 * tt - 1) / (8 * tt)));
    hippo::short_conv_fwd_vec_kernel<4><<<grid, 256, 0, ST(s)>>>((const bf16*)x, ldx, (const bf16*)w, pos, (bf16*)y, T, D, tt);
    RET();
  }
  long long n = T * D;
  hippo::short_conv_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ST(s)>>>((const bf16*)x, ldx, (const bf16*)w, pos, (bf16*)y, T, D, W);
  RET();
}
extern "C" int hippo_short_conv_bwd(const void* x, long long ldx, const void* w, const int* pos, const void* dy, void* dx,
                                    long long lddx, float* dw, long long T, int D, int W, void* s) {
  if (W > 8) return -1;
  if (T <= 0 || D <= 0) return 0;
  if (W == 4 && D % 8 == 0 && ldx % 8 == 0 && lddx % 8 == 0 && !((uintptr_t)x & 15) && !((uintptr_t)dy & 15) &&
      !((uintptr_t)dx & 15)) {
    const int tt = 32;
    dim3 grid((D / 8 + 31) / 32, (unsigned)((T + 8 * tt - 1) / (8 * tt)));
    hippo::short_conv_bwd_vec_kernel<4><<<grid, 256, 0, ST(s)>>>((const bf16*)x, ldx, (const bf16*)w, pos, (const bf16*)dy,
                                                                 (bf16*)dx, lddx, dw, T, D, tt);
    RET();
  }
  dim3 grid((D + 127) / 128, (unsigned)(T < 64 ? 1 : (T / 64 > 512 ? 512 : T / 64)));
  hippo::short_conv_bwd_kernel<<<grid, 128, 0, ST(s)>>>((const bf16*)x, ldx, (const bf16*)w, pos, (const bf16*)dy, (bf16*)dx, lddx, dw, T, D, W);
  RET();
}
