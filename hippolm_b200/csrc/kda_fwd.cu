// Chunked Kimi-Delta-Attention forward (chunk = 64 tokens, K = V = DK in {64, 128}).
//
// kda_fwd_intra  one CTA per (chunk, head): inclusive cumsum G of the log decay, the decayed Gram
//                matrices kk/qk, (I + beta*kk)^-1 by blocked forward substitution, then
//                w = Ainv (beta k e^G), u = Ainv (beta v), qg = q e^G, kg = k e^(Glast-G).
//                Pairwise decays exp(G_i - G_j) are factorised around a sub-chunk anchor so that both
//                factors are <= 1 for any decay magnitude (16x16 diagonal blocks are formed exactly).
// kda_fwd_state  one CTA per (sequence, head, 32-column slice of V): sequential over the chunks of
//                the sequence with the K x 32 state slice resident in shared memory:
//                v_new = u - w S;  o = qg S + Aqk v_new;  S <- e^Glast S + kg^T v_new.
// Replaces the reference's Triton pipeline (fla/ops/kda/chunk_fwd.py:43-135, chunk_intra.py:41-747,
// wy_fast.py:32-119, fla/ops/common/chunk_delta_h.py:40-323, fla/ops/gla/chunk.py:313-392).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <mma.h>
#include <stdint.h>
#include "kda_common.cuh"
#include <stdlib.h>

namespace hippo {
using namespace nvcuda;

// Bytes of the intra kernel's work region: phase 2 holds two 48-row operand tiles and a 16-row column tile there,
// phases 3-4 the fp32 inverse (pitch 68), three 16x16 fp32 temporaries and the bf16 copy of the inverse (pitch 72).
template <int DK>
__host__ __device__ constexpr int kda_intra_work_bytes() {
  constexpr int tiles = (2 * 48 + 16) * (DK + 8) * 2, inv = (64 * 68 + 3 * 256) * 4 + 64 * 72 * 2;
  return tiles > inv ? tiles : inv;
}

template <int DK>
__global__ void __launch_bounds__(512, 2)
kda_fwd_intra_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                     const float* __restrict__ g, const float* __restrict__ beta,
                     const int* __restrict__ chunk_start, const int* __restrict__ chunk_len, int H,
                     float* __restrict__ Gout, bf16* __restrict__ w_out, bf16* __restrict__ u_out,
                     bf16* __restrict__ qg_out, bf16* __restrict__ kg_out, bf16* __restrict__ Aqk_out,
                     bf16* __restrict__ Ainv_out, bf16* __restrict__ Akk_out) {
  constexpr int LD = DK + 8;       // bf16 tile pitch
  constexpr int LA = 68;           // fp32 pitch of the inverse X
  constexpr int LK = 64;           // fp32 pitch of kk / Akk
  constexpr int LG = DK + 4;       // fp32 G pitch (rows land on different banks); pad column DK holds beta
  // 113 KB at DK = 128, so that two CTAs share an SM: the chain of block-wide phases of one chunk is latency-bound
  // and the second CTA fills its barrier stalls.
  extern __shared__ __align__(128) uint8_t smem[];
  float* Gs = (float*)smem;                       // [64][LG]
  bf16* qs = (bf16*)(Gs + 64 * LG);               // [64][LD] q; phase 4 overwrites it in place with beta*v
  bf16* ks = qs + 64 * LD;                        // [64][LD] k; phase 4 overwrites it in place with beta*k*e^G
  uint8_t* work = (uint8_t*)(ks + 64 * LD);       // kda_intra_work_bytes<DK>()
  bf16* T1 = (bf16*)work;                         // [48][LD] phase 2 row side q * decay
  bf16* T2 = T1 + 48 * LD;                        // [48][LD] phase 2 row side k * decay
  bf16* Ck = T2 + 48 * LD;                        // [16][LD] phase 2 column side
  // phases 3 and 4 reuse the work region, which is idle after phase 2
  float* X = (float*)work;                        // [64][LA]
  float* Tm = X + 64 * LA;                        // [3][16][16]
  bf16* Xb = (bf16*)(Tm + 3 * 256);               // [64][72]
  constexpr int WORK = kda_intra_work_bytes<DK>();
  float* kk = (float*)(work + WORK);              // [64][LK]
  float* bs = Gs + DK;                            // beta of row i at bs[i * LG]

  constexpr int NTHR = 512, NWARP = 16;
  const int chunk = blockIdx.x, h = blockIdx.y;
  const int t0 = chunk_start[chunk], len = chunk_len[chunk];
  if (len == 0) return;                                       // padding entry of the chunk table
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long cbase = ((long long)chunk * H + h) * 64;   // row base in chunk-padded [NC,H,64,*] arrays

  // ---- phase 0: loads, cumsum
  for (int idx = tid; idx < 64 * (DK / 8); idx += NTHR) {
    int r = idx / (DK / 8), c8 = (idx % (DK / 8)) * 8;
    uint4 zq = make_uint4(0, 0, 0, 0), zk = zq;
    if (r < len) {
      long long off = ((long long)(t0 + r) * H + h) * DK + c8;
      zq = *(const uint4*)(q + off); zk = *(const uint4*)(k + off);
    }
    *(uint4*)(qs + r * LD + c8) = zq; *(uint4*)(ks + r * LD + c8) = zk;
  }
  for (int idx = tid; idx < 64 * LK; idx += NTHR) kk[idx] = 0.f;
  if (tid < 64) bs[tid * LG] = tid < len ? beta[(long long)(t0 + tid) * H + h] : 0.f;
  if (tid < DK) {
    float run = 0.f;
#pragma unroll 8
    for (int r = 0; r < 64; ++r) {
      float gv = r < len ? g[((long long)(t0 + r) * H + h) * DK + tid] : 0.f;
      run += gv;
      Gs[r * LG + tid] = run;
      Gout[(cbase + r) * DK + tid] = run;
    }
  }
  __syncthreads();

  // ---- phase 1: exact diagonal 16x16 blocks. 8-lane groups, each lane owns DK/8 channels.
  {
    constexpr int CPL = DK / 8;
    const int grp = tid >> 3, gl = tid & 7;
    for (int p0 = grp; p0 < 4 * 136 + 32; p0 += NTHR / 8) {     // uniform trip count: shuffles need every lane
      const bool valid = p0 < 4 * 136;
      const int p = valid ? p0 : 0;
      int b = p / 136, r = p % 136;
      int ii = 0;
      while ((ii + 1) * (ii + 2) / 2 <= r) ++ii;
      int jj = r - ii * (ii + 1) / 2;
      int i = b * 16 + ii, j = b * 16 + jj;
      float skk = 0.f, sqk = 0.f;
      // lane gl owns channels 32 m + 4 gl .. + 3: one float4 / uint2 per operand and group, conflict-free across the 8 lanes
#pragma unroll
      for (int m = 0; m < CPL / 4; ++m) {
        const int c = m * 32 + gl * 4;
        const float4 gi = *(const float4*)(Gs + i * LG + c), gj = *(const float4*)(Gs + j * LG + c);
        const uint2 kiw = *(const uint2*)(ks + i * LD + c), kjw = *(const uint2*)(ks + j * LD + c), qiw = *(const uint2*)(qs + i * LD + c);
        const float2 ki0 = __bfloat1622float2(*(const __nv_bfloat162*)&kiw.x), ki1 = __bfloat1622float2(*(const __nv_bfloat162*)&kiw.y);
        const float2 kj0 = __bfloat1622float2(*(const __nv_bfloat162*)&kjw.x), kj1 = __bfloat1622float2(*(const __nv_bfloat162*)&kjw.y);
        const float2 qi0 = __bfloat1622float2(*(const __nv_bfloat162*)&qiw.x), qi1 = __bfloat1622float2(*(const __nv_bfloat162*)&qiw.y);
        float t;
        t = kj0.x * __expf(gi.x - gj.x); skk += ki0.x * t; sqk += qi0.x * t;
        t = kj0.y * __expf(gi.y - gj.y); skk += ki0.y * t; sqk += qi0.y * t;
        t = kj1.x * __expf(gi.z - gj.z); skk += ki1.x * t; sqk += qi1.x * t;
        t = kj1.y * __expf(gi.w - gj.w); skk += ki1.y * t; sqk += qi1.y * t;
      }
      skk += __shfl_xor_sync(0xFFFFFFFFu, skk, 1); sqk += __shfl_xor_sync(0xFFFFFFFFu, sqk, 1);
      skk += __shfl_xor_sync(0xFFFFFFFFu, skk, 2); sqk += __shfl_xor_sync(0xFFFFFFFFu, sqk, 2);
      skk += __shfl_xor_sync(0xFFFFFFFFu, skk, 4); sqk += __shfl_xor_sync(0xFFFFFFFFu, sqk, 4);
      if (gl == 0 && valid) { if (jj < ii) kk[i * LK + j] = skk; Aqk_out[(cbase + i) * 64 + j] = __float2bfloat16(sqk); }
    }
  }

  // ---- phase 2: off-diagonal blocks, column block J anchored at its last row
  for (int J = 0; J < 3; ++J) {
    const int e = 16 * J + 15, r0 = 16 * (J + 1), nrows = 64 - r0;
    __syncthreads();
    for (int idx = tid; idx < 16 * DK; idx += NTHR) {
      int jj = idx / DK, c = idx % DK, j = 16 * J + jj;
      Ck[jj * LD + c] = __float2bfloat16(__bfloat162float(ks[j * LD + c]) * __expf(Gs[e * LG + c] - Gs[j * LG + c]));
    }
    for (int idx = tid; idx < nrows * DK; idx += NTHR) {
      int rr = idx / DK, c = idx % DK, i = r0 + rr;
      float f = __expf(Gs[i * LG + c] - Gs[e * LG + c]);
      T1[rr * LD + c] = __float2bfloat16(__bfloat162float(qs[i * LD + c]) * f);
      T2[rr * LD + c] = __float2bfloat16(__bfloat162float(ks[i * LD + c]) * f);
    }
    __syncthreads();
    const int ntile = 2 * (nrows / 16);
    if (warp < ntile) {
      const int rt = warp >> 1, which = warp & 1;
      const bf16* R = which ? T2 : T1;
      const int g = lane >> 2, t4 = lane & 3;
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kt = 0; kt < DK / 16; ++kt) {
        unsigned a[4], b[4];
        kda_frag_a(a, R, LD, rt * 16, kt * 16, lane);
        kda_frag_bt2(b, Ck, LD, 0, kt * 16, lane);                  // Ck^T: n = column-block row, k = channel
        kda_mma16816(acc[0], a, b[0], b[1]);
        kda_mma16816(acc[1], a, b[2], b[3]);
      }
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int i = r0 + rt * 16 + g + hh * 8, j = 16 * J + n * 8 + 2 * t4;
          if (which) *(float2*)(kk + i * LK + j) = make_float2(acc[n][2 * hh], acc[n][2 * hh + 1]);
          else *(unsigned*)(Aqk_out + (cbase + i) * 64 + j) = kda_pack2(acc[n][2 * hh], acc[n][2 * hh + 1]);
        }
    }
  }
  __syncthreads();

  // ---- phase 3: X = (I + beta*kk)^-1, blocked forward substitution in fp32
  for (int idx = tid; idx < 64 * 64; idx += NTHR) {
    int i = idx >> 6, j = idx & 63;
    kk[i * LK + j] = j < i ? kk[i * LK + j] * bs[i * LG] : 0.f;      // kk now holds Akk
    X[i * LA + j] = 0.f;
  }
  __syncthreads();
  if (tid < 64) {
    const int b = tid >> 4, col = tid & 15;
    float x[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      float s = (r == col) ? 1.f : 0.f;
#pragma unroll
      for (int m = 0; m < 16; ++m)
        if (m < r) s -= kk[(b * 16 + r) * LK + b * 16 + m] * x[m];
      x[r] = s;
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) X[(b * 16 + r) * LA + b * 16 + col] = x[r];
  }
  __syncthreads();
  {
    const int r = (tid >> 4) & 15, c = tid & 15;
    const bool act = tid < 256;
    for (int d = 1; d < 4; ++d) {
      for (int J = 0; J + d < 4 && act; ++J) {
        const int I = J + d;
        float s = 0.f;
        for (int L = J; L < I; ++L)
#pragma unroll
          for (int m = 0; m < 16; ++m) s += kk[(I * 16 + r) * LK + L * 16 + m] * X[(L * 16 + m) * LA + J * 16 + c];
        Tm[J * 256 + r * 16 + c] = s;
      }
      __syncthreads();
      for (int J = 0; J + d < 4 && act; ++J) {
        const int I = J + d;
        float s = 0.f;
#pragma unroll
        for (int m = 0; m < 16; ++m) s += X[(I * 16 + r) * LA + I * 16 + m] * Tm[J * 256 + m * 16 + c];
        X[(I * 16 + r) * LA + J * 16 + c] = -s;
      }
      __syncthreads();
    }
  }

  // ---- phase 4: operands + outputs. The B operands of the two products overwrite k and q in place (every element is
  // read and written by the same thread), so no barrier separates the two loops.
  for (int idx = tid; idx < 64 * 64; idx += NTHR) {
    int i = idx >> 6, j = idx & 63;
    bf16 xv = __float2bfloat16(X[i * LA + j]);
    Xb[i * 72 + j] = xv;
    Ainv_out[(cbase + i) * 64 + j] = xv;
    Akk_out[(cbase + i) * 64 + j] = __float2bfloat16(kk[i * LK + j]);
    if (j > i) Aqk_out[(cbase + i) * 64 + j] = __float2bfloat16(0.f);
  }
  for (int idx = tid; idx < 64 * (DK / 8); idx += NTHR) {
    const int i = idx / (DK / 8), c8 = (idx % (DK / 8)) * 8;
    uint4 vq = make_uint4(0, 0, 0, 0);
    if (i < len) vq = *(const uint4*)(v + ((long long)(t0 + i) * H + h) * DK + c8);
    const uint4 kq = *(const uint4*)(ks + i * LD + c8), qq = *(const uint4*)(qs + i * LD + c8);
    const __nv_bfloat162* kb = (const __nv_bfloat162*)&kq; const __nv_bfloat162* qb = (const __nv_bfloat162*)&qq;
    const __nv_bfloat162* vb = (const __nv_bfloat162*)&vq;
    uint4 o1, o2, oq, ok;
    unsigned* w1 = (unsigned*)&o1; unsigned* w2 = (unsigned*)&o2; unsigned* wq = (unsigned*)&oq; unsigned* wk = (unsigned*)&ok;
    const float b = bs[i * LG];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int c = c8 + 2 * e;
      const float G0 = Gs[i * LG + c], G1 = Gs[i * LG + c + 1];
      const float e0 = __expf(G0), e1 = __expf(G1);
      const float2 kf = __bfloat1622float2(kb[e]), qf = __bfloat1622float2(qb[e]), vf = __bfloat1622float2(vb[e]);
      w1[e] = kda_pack2(b * kf.x * e0, b * kf.y * e1);
      w2[e] = kda_pack2(b * vf.x, b * vf.y);
      wq[e] = kda_pack2(qf.x * e0, qf.y * e1);
      wk[e] = kda_pack2(kf.x * __expf(Gs[63 * LG + c] - G0), kf.y * __expf(Gs[63 * LG + c + 1] - G1));
    }
    *(uint4*)(ks + i * LD + c8) = o1;
    *(uint4*)(qs + i * LD + c8) = o2;
    *(uint4*)(qg_out + (cbase + i) * DK + c8) = oq;
    *(uint4*)(kg_out + (cbase + i) * DK + c8) = ok;
  }
  __syncthreads();
  {
    // w = X (beta k e^G), u = X (beta v): warp (which, rt, column half) owns a 16-row x (DK/2)-column slab
    static_assert(NWARP == 16, "slab assignment below assumes 16 warps");
    const int which = warp >> 3, rt = (warp >> 1) & 3, ch = warp & 1;
    const bf16* B = which ? qs : ks;
    bf16* out = which ? u_out : w_out;
    const int g = lane >> 2, t4 = lane & 3;
    constexpr int NP = DK / 32;                       // pairs of n-tiles in half of the columns
    float acc[2 * NP][4];
#pragma unroll
    for (int n = 0; n < 2 * NP; ++n) { acc[n][0] = 0.f; acc[n][1] = 0.f; acc[n][2] = 0.f; acc[n][3] = 0.f; }
    for (int kt = 0; kt <= rt; ++kt) {                // X is lower triangular
      unsigned a[4];
      kda_frag_a(a, Xb, 72, rt * 16, kt * 16, lane);
#pragma unroll
      for (int np = 0; np < NP; ++np) {
        unsigned b[4];
        kda_frag_b2(b, B, LD, kt * 16, ch * (DK / 2) + np * 16, lane);
        kda_mma16816(acc[2 * np], a, b[0], b[1]);
        kda_mma16816(acc[2 * np + 1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int n = 0; n < 2 * NP; ++n)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        *(unsigned*)(out + (cbase + rt * 16 + g + hh * 8) * DK + ch * (DK / 2) + n * 8 + 2 * t4) =
            kda_pack2(acc[n][2 * hh], acc[n][2 * hh + 1]);
  }
}

template <int DK>
constexpr int kda_intra_smem() {
  return 64 * (DK + 4) * 4 + 2 * 64 * (DK + 8) * 2 + kda_intra_work_bytes<DK>() + 64 * 64 * 4;
}
static_assert(2 * (kda_intra_smem<128>() + 1024) <= 228 * 1024, "two CTAs of the intra kernel must fit one SM");

// ---------------------------------------------------------------------------------------------------
// 256 threads, one CTA per SM. The tiles of chunk n+1 stream into the second shared-memory buffer with cp.async
// while chunk n is computed, so the global load latency is off the sequential critical path (the chain over
// chunks is what bounds this kernel).
template <int DK, int VS>
__global__ void __launch_bounds__(256, 1)
kda_fwd_state_kernel(const bf16* __restrict__ w, const bf16* __restrict__ u, const bf16* __restrict__ qg,
                     const bf16* __restrict__ kg, const bf16* __restrict__ Aqk, const float* __restrict__ G,
                     const int* __restrict__ chunk_start, const int* __restrict__ chunk_len,
                     const int* __restrict__ seq_chunk, const int* __restrict__ seq_order, int H,
                     const float* __restrict__ h0, bf16* __restrict__ vnew_out, bf16* __restrict__ S_out,
                     bf16* __restrict__ o, float* __restrict__ final_state) {
  constexpr int LD = DK + 8, LS = VS + 8, LF = VS + 4, NTHR = 256;
  constexpr int NV_BIG = 64 * (DK / 8) / NTHR;          // uint4 per thread for one [64, DK] tile
  constexpr int NV_AQ = 64 * 8 / NTHR;                   // Aqk tile
  static_assert(64 * (VS / 8) <= NTHR && DK <= NTHR, "tile/thread mapping");
  extern __shared__ __align__(128) uint8_t smem[];
  float* S = (float*)smem;                    // [DK][LF]
  float* stg = S + DK * LF;                   // [64][LF]
  float* egl = stg + 64 * LF;                 // [DK]
  bf16* Sb = (bf16*)(egl + DK);               // [DK][LS]
  bf16* vns = Sb + DK * LS;                   // [64][LS]
  bf16* tiles = vns + 64 * LS;                // 2 x { w, qg, kg: [64][LD] ; Aqk: [64][72] ; u: [64][LS] ; Glast: DK floats }
  constexpr int TILE_ELEMS = 3 * 64 * LD + 64 * 72 + 64 * LS + 2 * DK;

  const int vs0 = blockIdx.x * VS, h = blockIdx.y, seq = seq_order[blockIdx.z];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c_begin = seq_chunk[seq], c_end = seq_chunk[seq + 1];

  for (int idx = tid; idx < DK * VS; idx += NTHR) {
    int r = idx / VS, c = idx % VS;
    float s0 = h0 ? h0[(((long long)seq * H + h) * DK + r) * DK + vs0 + c] : 0.f;
    S[r * LF + c] = s0;
    Sb[r * LS + c] = __float2bfloat16(s0);
  }
  auto fetch = [&](int chunk, int buf) {
    const long long cbase = ((long long)chunk * H + h) * 64;
    bf16* tb = tiles + buf * TILE_ELEMS;
    bf16* ws_ = tb; bf16* qgs_ = ws_ + 64 * LD; bf16* kgs_ = qgs_ + 64 * LD; bf16* Aq_ = kgs_ + 64 * LD;
    bf16* us_ = Aq_ + 64 * 72; float* gl_ = (float*)(us_ + 64 * LS);
#pragma unroll
    for (int j = 0; j < NV_BIG; ++j) {
      int idx = tid + j * NTHR, r = idx / (DK / 8), c8 = (idx % (DK / 8)) * 8;
      long long off = (cbase + r) * DK + c8;
      cp_async16(ws_ + r * LD + c8, w + off); cp_async16(qgs_ + r * LD + c8, qg + off); cp_async16(kgs_ + r * LD + c8, kg + off);
    }
#pragma unroll
    for (int j = 0; j < NV_AQ; ++j) {
      int idx = tid + j * NTHR, r = idx >> 3, c8 = (idx & 7) * 8;
      cp_async16(Aq_ + r * 72 + c8, Aqk + (cbase + r) * 64 + c8);
    }
    if (tid < 64 * (VS / 8)) {
      int r = tid / (VS / 8), c8 = (tid % (VS / 8)) * 8;
      cp_async16(us_ + r * LS + c8, u + (cbase + r) * DK + vs0 + c8);
    }
    if (tid < DK / 4) cp_async16(gl_ + tid * 4, G + (cbase + 63) * DK + tid * 4);
    cp_async_commit();
  };
  if (c_begin < c_end) fetch(c_begin, 0);
  __syncthreads();

  for (int chunk = c_begin; chunk < c_end; ++chunk) {
    const long long cbase = ((long long)chunk * H + h) * 64;
    const int t0 = chunk_start[chunk], len = chunk_len[chunk];
    const int buf = (chunk - c_begin) & 1;
    bf16* ws = tiles + buf * TILE_ELEMS; bf16* qgs = ws + 64 * LD; bf16* kgs = qgs + 64 * LD; bf16* Aq = kgs + 64 * LD;
    bf16* us = Aq + 64 * 72; const float* gl = (const float*)(us + 64 * LS);
    cp_async_wait_all();
    __syncthreads();                                        // this chunk's tiles have landed; the other buffer is free
    if (chunk + 1 < c_end) fetch(chunk + 1, buf ^ 1);       // in flight during the math below
    if (tid < 64 * (VS / 8)) {
      int r = tid / (VS / 8), c8 = (tid % (VS / 8)) * 8;
      *(uint4*)(vns + r * LS + c8) = *(const uint4*)(us + r * LS + c8);
    }
    if (tid < DK) egl[tid] = __expf(gl[tid]);
    // state at chunk start, for the backward pass
    for (int idx = tid; idx < DK * (VS / 8); idx += NTHR) {
      int r = idx / (VS / 8), c8 = (idx % (VS / 8)) * 8;
      *(uint4*)(S_out + (((long long)chunk * H + h) * DK + r) * DK + vs0 + c8) = *(const uint4*)(Sb + r * LS + c8);
    }
    __syncthreads();

    // P = w S ; v_new = u - P      (8 warps: 4 row tiles x VS/16 column tiles)
    const int rt = warp % 4, nt0 = warp / 4;              // VS/16 == 2 column tiles
    {
      wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
      wmma::fill_fragment(acc, 0.f);
#pragma unroll
      for (int kt = 0; kt < DK / 16; ++kt) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
        wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> b;
        wmma::load_matrix_sync(a, ws + rt * 16 * LD + kt * 16, LD);
        wmma::load_matrix_sync(b, Sb + kt * 16 * LS + nt0 * 16, LS);
        wmma::mma_sync(acc, a, b, acc);
      }
      wmma::store_matrix_sync(stg + rt * 16 * LF + nt0 * 16, acc, LF, wmma::mem_row_major);
      __syncwarp();
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int el = lane * 8 + e, rr = rt * 16 + (el >> 4), cc = nt0 * 16 + (el & 15);
        float vn = __bfloat162float(vns[rr * LS + cc]) - stg[rr * LF + cc];
        bf16 vb = __float2bfloat16(vn);
        vns[rr * LS + cc] = vb;
        vnew_out[(cbase + rr) * DK + vs0 + cc] = vb;
      }
    }
    __syncthreads();
    // o = qg S + Aqk v_new
    {
      wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
      wmma::fill_fragment(acc, 0.f);
#pragma unroll
      for (int kt = 0; kt < DK / 16; ++kt) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
        wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> b;
        wmma::load_matrix_sync(a, qgs + rt * 16 * LD + kt * 16, LD);
        wmma::load_matrix_sync(b, Sb + kt * 16 * LS + nt0 * 16, LS);
        wmma::mma_sync(acc, a, b, acc);
      }
      for (int kt = 0; kt <= rt; ++kt) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
        wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> b;
        wmma::load_matrix_sync(a, Aq + rt * 16 * 72 + kt * 16, 72);
        wmma::load_matrix_sync(b, vns + kt * 16 * LS + nt0 * 16, LS);
        wmma::mma_sync(acc, a, b, acc);
      }
      wmma::store_matrix_sync(stg + rt * 16 * LF + nt0 * 16, acc, LF, wmma::mem_row_major);
      __syncwarp();
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int el = lane * 8 + e, rr = rt * 16 + (el >> 4), cc = nt0 * 16 + (el & 15);
        if (rr < len) o[((long long)(t0 + rr) * H + h) * DK + vs0 + cc] = __float2bfloat16(stg[rr * LF + cc]);
      }
    }
    __syncthreads();                                       // every warp is done reading Sb
    // S <- e^Glast S + kg^T v_new   (each warp owns its tiles: scale, accumulate, write S and the bf16 copy)
    for (int t = warp; t < (DK / 16) * (VS / 16); t += 8) {
      const int mt = t / (VS / 16), nt = t % (VS / 16);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int el = lane * 8 + e, rr = mt * 16 + (el >> 4), cc = nt * 16 + (el & 15);
        S[rr * LF + cc] *= egl[rr];
      }
      __syncwarp();
      wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
      wmma::load_matrix_sync(acc, S + mt * 16 * LF + nt * 16, LF, wmma::mem_row_major);
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::col_major> a;     // kg^T
        wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> b;
        wmma::load_matrix_sync(a, kgs + kt * 16 * LD + mt * 16, LD);
        wmma::load_matrix_sync(b, vns + kt * 16 * LS + nt * 16, LS);
        wmma::mma_sync(acc, a, b, acc);
      }
      wmma::store_matrix_sync(S + mt * 16 * LF + nt * 16, acc, LF, wmma::mem_row_major);
      __syncwarp();
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int el = lane * 8 + e, rr = mt * 16 + (el >> 4), cc = nt * 16 + (el & 15);
        Sb[rr * LS + cc] = __float2bfloat16(S[rr * LF + cc]);
      }
    }
    __syncthreads();
  }
  if (final_state) {
    for (int idx = tid; idx < DK * VS; idx += NTHR) {
      int r = idx / VS, c = idx % VS;
      final_state[(((long long)seq * H + h) * DK + r) * DK + vs0 + c] = S[r * LF + c];
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Register-resident variant of the state recurrence for DK = 128 (mma.sync m16n8k16 + ldmatrix).
// The chain over chunks is what bounds this kernel, so everything is arranged around its critical path
//     S(t) -> P = w S -> v_new = u - P -> S(t+1) = e^Glast S + kg^T v_new
// * the fp32 state never leaves registers: warp w owns rows 16w..16w+15 of the [128 x VS] slice (16 values per thread);
//   only its bf16 image goes to shared memory as the B operand of the next chunk;
// * the output product o = qg S + Aqk v_new is not on the chain, so it runs AFTER the state update, reusing the
//   B fragments of S it kept from the P product; the next chunk's P product of faster warps overlaps it;
// * two barriers per chunk; tiles arrive by cp.async in two double-buffered sets with different lifetimes
//   ({w, u, kg, Glast} until the state update, {qg, Aqk} until the deferred output product).
template <int VS>
__global__ void __launch_bounds__(256, 1)
kda_fwd_state_mma_kernel(const bf16* __restrict__ w, const bf16* __restrict__ u, const bf16* __restrict__ qg,
                         const bf16* __restrict__ kg, const bf16* __restrict__ Aqk, const float* __restrict__ G,
                         const int* __restrict__ chunk_start, const int* __restrict__ chunk_len,
                         const int* __restrict__ seq_chunk, const int* __restrict__ seq_order, int H,
                         const float* __restrict__ h0, bf16* __restrict__ vnew_out, bf16* __restrict__ S_out,
                         bf16* __restrict__ o, float* __restrict__ final_state) {
  constexpr int DK = 128, LD = DK + 8, LS = VS + 8, LQ = 72, NTHR = 256;
  static_assert(VS == 32, "warp tiling below assumes a 32-column value slice");
  constexpr int SETA = 2 * 64 * LD + 64 * LS + 2 * DK;       // bf16 elements: w, kg, u, Glast (DK floats)
  constexpr int SETB = 64 * LD + 64 * LQ;                    // qg, Aqk
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* setA = (bf16*)smem;                                  // 2 x SETA
  bf16* setB = setA + 2 * SETA;                              // 2 x SETB
  bf16* Sb = setB + 2 * SETB;                                // [DK][LS] bf16 image of the state
  bf16* vns = Sb + DK * LS;                                  // 2 x [64][LS]
  float* egl = (float*)(vns + 2 * 64 * LS);                  // [DK]

  const int vs0 = blockIdx.x * VS, h = blockIdx.y, seq = seq_order[blockIdx.z];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int c_begin = seq_chunk[seq], c_end = seq_chunk[seq + 1];
  if (c_begin >= c_end) return;
  const int mt = warp & 3, nh = warp >> 2;                   // P / o products: 16-row tile mt, 16-column half nh
  const int srow = warp * 16 + g;                            // state rows of this thread: srow, srow + 8

  float S[4][4];                                             // [n-tile][c0..c3]
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int c = vs0 + nt * 8 + 2 * t4;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = srow + (e >> 1) * 8;
      S[nt][e] = h0 ? h0[(((long long)seq * H + h) * DK + r) * DK + c + (e & 1)] : 0.f;
    }
    *(unsigned*)(Sb + srow * LS + nt * 8 + 2 * t4) = kda_pack2(S[nt][0], S[nt][1]);
    *(unsigned*)(Sb + (srow + 8) * LS + nt * 8 + 2 * t4) = kda_pack2(S[nt][2], S[nt][3]);
  }
  auto fetchA = [&](int chunk, int buf) {
    const long long cbase = ((long long)chunk * H + h) * 64;
    bf16* ws_ = setA + buf * SETA; bf16* kgs_ = ws_ + 64 * LD; bf16* us_ = kgs_ + 64 * LD; float* gl_ = (float*)(us_ + 64 * LS);
#pragma unroll
    for (int j = 0; j < 64 * (DK / 8) / NTHR; ++j) {
      const int idx = tid + j * NTHR, r = idx >> 4, c8 = (idx & 15) * 8;
      const long long off = (cbase + r) * DK + c8;
      cp_async16(ws_ + r * LD + c8, w + off); cp_async16(kgs_ + r * LD + c8, kg + off);
    }
    { const int r = tid >> 2, c8 = (tid & 3) * 8; cp_async16(us_ + r * LS + c8, u + (cbase + r) * DK + vs0 + c8); }
    if (tid < DK / 4) cp_async16(gl_ + tid * 4, G + (cbase + 63) * DK + tid * 4);
  };
  auto fetchB = [&](int chunk, int buf) {
    const long long cbase = ((long long)chunk * H + h) * 64;
    bf16* qgs_ = setB + buf * SETB; bf16* Aq_ = qgs_ + 64 * LD;
#pragma unroll
    for (int j = 0; j < 64 * (DK / 8) / NTHR; ++j) {
      const int idx = tid + j * NTHR, r = idx >> 4, c8 = (idx & 15) * 8;
      cp_async16(qgs_ + r * LD + c8, qg + (cbase + r) * DK + c8);
    }
#pragma unroll
    for (int j = 0; j < 64 * 8 / NTHR; ++j) {
      const int idx = tid + j * NTHR, r = idx >> 3, c8 = (idx & 7) * 8;
      cp_async16(Aq_ + r * LQ + c8, Aqk + (cbase + r) * 64 + c8);
    }
  };
  fetchA(c_begin, 0); cp_async_commit();
  fetchB(c_begin, 0); cp_async_commit();
  cp_async_wait_all();
  __syncthreads();

  for (int chunk = c_begin; chunk < c_end; ++chunk) {
    const long long cbase = ((long long)chunk * H + h) * 64;
    const int t0 = chunk_start[chunk], len = chunk_len[chunk];
    const int a = (chunk - c_begin) & 1;
    const bf16* ws = setA + a * SETA; const bf16* kgs = ws + 64 * LD; const bf16* us = kgs + 64 * LD;
    const float* gl = (const float*)(us + 64 * LS);
    const bf16* qgs = setB + a * SETB; const bf16* Aq = qgs + 64 * LD;
    bf16* vn = vns + a * 64 * LS;

    if (chunk + 1 < c_end) fetchA(chunk + 1, a ^ 1);          // set A of the previous chunk was released at its last barrier
    cp_async_commit();
    if (tid < DK) egl[tid] = __expf(gl[tid]);
    // state at chunk start, for the backward pass
#pragma unroll
    for (int j = 0; j < DK * (VS / 8) / NTHR; ++j) {
      const int idx = tid + j * NTHR, r = idx / (VS / 8), c8 = (idx % (VS / 8)) * 8;
      *(uint4*)(S_out + (((long long)chunk * H + h) * DK + r) * DK + vs0 + c8) = *(const uint4*)(Sb + r * LS + c8);
    }

    // ---- P = w S (rows mt*16.., columns nh*16..), v_new = u - P. The B fragments of S are kept for the output product.
    unsigned bS[8][4];
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      unsigned af[4];
      kda_frag_a(af, ws, LD, mt * 16, kk * 16, lane);
      kda_frag_b2(bS[kk], Sb, LS, kk * 16, nh * 16, lane);
      kda_mma16816(acc[0], af, bS[kk][0], bS[kk][1]);
      kda_mma16816(acc[1], af, bS[kk][2], bS[kk][3]);
    }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const int c = nh * 16 + nt * 8 + 2 * t4;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int r = mt * 16 + g + hh * 8;
        const float2 uv = __bfloat1622float2(*(const __nv_bfloat162*)(us + r * LS + c));
        const unsigned pk = kda_pack2(uv.x - acc[nt][2 * hh], uv.y - acc[nt][2 * hh + 1]);
        *(unsigned*)(vn + r * LS + c) = pk;
        *(unsigned*)(vnew_out + (cbase + r) * DK + vs0 + c) = pk;
      }
    }
    __syncthreads();                                          // v_new complete; every warp is past its reads of Sb
    if (chunk + 1 < c_end) fetchB(chunk + 1, a ^ 1);          // set B of the previous chunk: its output product is done
    cp_async_commit();

    // ---- S <- e^Glast S + kg^T v_new   (this warp's 16 state rows, all VS columns)
    {
      const float e0 = egl[srow], e1 = egl[srow + 8];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) { S[nt][0] *= e0; S[nt][1] *= e0; S[nt][2] *= e1; S[nt][3] *= e1; }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        unsigned af[4], b0[4], b1[4];
        kda_frag_a_t(af, kgs, LD, warp * 16, kk * 16, lane);
        kda_frag_b2(b0, vn, LS, kk * 16, 0, lane);
        kda_frag_b2(b1, vn, LS, kk * 16, 16, lane);
        kda_mma16816(S[0], af, b0[0], b0[1]);
        kda_mma16816(S[1], af, b0[2], b0[3]);
        kda_mma16816(S[2], af, b1[0], b1[1]);
        kda_mma16816(S[3], af, b1[2], b1[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        *(unsigned*)(Sb + srow * LS + nt * 8 + 2 * t4) = kda_pack2(S[nt][0], S[nt][1]);
        *(unsigned*)(Sb + (srow + 8) * LS + nt * 8 + 2 * t4) = kda_pack2(S[nt][2], S[nt][3]);
      }
    }
    cp_async_wait_group<1>();                                 // next chunk's set A (and this chunk's set B) have landed
    __syncthreads();

    // ---- o = qg S(chunk start) + Aqk v_new   (off the chain: uses the kept fragments of S)
    {
      float oc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        unsigned af[4];
        kda_frag_a(af, qgs, LD, mt * 16, kk * 16, lane);
        kda_mma16816(oc[0], af, bS[kk][0], bS[kk][1]);
        kda_mma16816(oc[1], af, bS[kk][2], bS[kk][3]);
      }
      for (int kk = 0; kk <= mt; ++kk) {                      // Aqk is lower triangular in 16-row blocks
        unsigned af[4], bv[4];
        kda_frag_a(af, Aq, LQ, mt * 16, kk * 16, lane);
        kda_frag_b2(bv, vn, LS, kk * 16, nh * 16, lane);
        kda_mma16816(oc[0], af, bv[0], bv[1]);
        kda_mma16816(oc[1], af, bv[2], bv[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int c = nh * 16 + nt * 8 + 2 * t4;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = mt * 16 + g + hh * 8;
          if (r < len)
            *(unsigned*)(o + ((long long)(t0 + r) * H + h) * DK + vs0 + c) = kda_pack2(oc[nt][2 * hh], oc[nt][2 * hh + 1]);
        }
      }
    }
  }
  if (final_state) {
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int c = vs0 + nt * 8 + 2 * t4;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        *(float2*)(final_state + (((long long)seq * H + h) * DK + srow + hh * 8) * DK + c) = make_float2(S[nt][2 * hh], S[nt][2 * hh + 1]);
    }
  }
}

template <int VS>
constexpr int kda_state_mma_smem() {
  return (2 * (2 * 64 * 136 + 64 * (VS + 8) + 2 * 128) + 2 * (64 * 136 + 64 * 72) + 128 * (VS + 8) + 2 * 64 * (VS + 8)) * 2 + 128 * 4 + 128;
}

template <int DK, int VS>
constexpr int kda_state_smem() {
  return DK * (VS + 4) * 4 + 64 * (VS + 4) * 4 + DK * 4 + DK * (VS + 8) * 2 + 64 * (VS + 8) * 2 +
         2 * (3 * 64 * (DK + 8) + 64 * 72 + 64 * (VS + 8) + 2 * DK) * 2 + 128;
}

}  // namespace hippo

using namespace hippo;

// HIPPO_KDA_STATE_MMA=0 selects the WMMA state kernels for head_dim 128 as well (they always serve head_dim 64)
static bool kda_state_mma_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("HIPPO_KDA_STATE_MMA"); v = (e && e[0] == '0') ? 0 : 1; }
  return v == 1;
}

template <int DK>
static int launch_fwd(const void* q, const void* k, const void* v, const float* g, const float* beta,
                      const int* cs, const int* cl, const int* sc, const int* so, int NC, int N, int H, const float* h0,
                      float* G, void* w, void* u, void* qg, void* kg, void* Aqk, void* Ainv, void* Akk, void* vnew,
                      void* Sst, void* o, float* fin, cudaStream_t s) {
  constexpr int VS = 32;
  auto k1 = kda_fwd_intra_kernel<DK>;
  auto k2 = kda_fwd_state_kernel<DK, VS>;
  static bool once = false;
  if (!once) {
    cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_intra_smem<DK>());
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_state_smem<DK, VS>());
    if (e != cudaSuccess) return (int)e;
    once = true;
  }
  if (NC == 0) return 0;
  k1<<<dim3(NC, H), 512, kda_intra_smem<DK>(), s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, g, beta, cs, cl, H,
                                                    G, (bf16*)w, (bf16*)u, (bf16*)qg, (bf16*)kg, (bf16*)Aqk, (bf16*)Ainv, (bf16*)Akk);
  if (DK == 128 && kda_state_mma_enabled()) {
    auto k3 = kda_fwd_state_mma_kernel<VS>;
    static bool once3 = false;
    if (!once3) {
      cudaError_t e = cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_state_mma_smem<VS>());
      if (e != cudaSuccess) return (int)e;
      once3 = true;
    }
    k3<<<dim3(DK / VS, H, N), 256, kda_state_mma_smem<VS>(), s>>>((const bf16*)w, (const bf16*)u, (const bf16*)qg,
                                                                  (const bf16*)kg, (const bf16*)Aqk, G, cs, cl, sc, so, H, h0,
                                                                  (bf16*)vnew, (bf16*)Sst, (bf16*)o, fin);
    return (int)cudaGetLastError();
  }
  k2<<<dim3(DK / VS, H, N), 256, kda_state_smem<DK, VS>(), s>>>((const bf16*)w, (const bf16*)u, (const bf16*)qg,
                                                                (const bf16*)kg, (const bf16*)Aqk, G, cs, cl, sc, so, H, h0,
                                                                (bf16*)vnew, (bf16*)Sst, (bf16*)o, fin);
  return (int)cudaGetLastError();
}

// q,k,v: [T,H,DK] bf16 (q already scaled, q/k already normalised); g: [T,H,DK] fp32 log decay; beta: [T,H] fp32.
// chunk tables: chunk_start/len [NC], seq_chunk [N+1]. Workspaces are chunk-padded [NC,H,64,*].
extern "C" int hippo_kda_fwd(const void* q, const void* k, const void* v, const float* g, const float* beta,
                             const int* chunk_start, const int* chunk_len, const int* seq_chunk, const int* seq_order,
                             int NC, int N, int H, int DK, const float* h0, float* G, void* w, void* u, void* qg, void* kg, void* Aqk,
                             void* Ainv, void* Akk, void* vnew, void* Sst, void* o, float* final_state, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (DK == 128) return launch_fwd<128>(q, k, v, g, beta, chunk_start, chunk_len, seq_chunk, seq_order, NC, N, H, h0, G, w, u, qg, kg, Aqk, Ainv, Akk, vnew, Sst, o, final_state, s);
  if (DK == 64) return launch_fwd<64>(q, k, v, g, beta, chunk_start, chunk_len, seq_chunk, seq_order, NC, N, H, h0, G, w, u, qg, kg, Aqk, Ainv, Akk, vnew, Sst, o, final_state, s);
  return -1;
}

// Only the per-chunk kernel (gate cumsum, WY / A matrices): recomputes G, w, u, qg, kg, Aqk, Ainv, Akk from the inputs.
// Used by the backward pass when the forward was asked not to keep these tensors (activation-memory option).
template <int DK>
static int launch_fwd_intra(const void* q, const void* k, const void* v, const float* g, const float* beta, const int* cs,
                            const int* cl, int NC, int H, float* G, void* w, void* u, void* qg, void* kg, void* Aqk,
                            void* Ainv, void* Akk, cudaStream_t s) {
  auto k1 = kda_fwd_intra_kernel<DK>;
  static bool once = false;
  if (!once) {
    cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_intra_smem<DK>());
    if (e != cudaSuccess) return (int)e;
    once = true;
  }
  if (NC == 0) return 0;
  k1<<<dim3(NC, H), 512, kda_intra_smem<DK>(), s>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, g, beta, cs, cl, H,
                                                    G, (bf16*)w, (bf16*)u, (bf16*)qg, (bf16*)kg, (bf16*)Aqk, (bf16*)Ainv, (bf16*)Akk);
  return (int)cudaGetLastError();
}

extern "C" int hippo_kda_fwd_intra(const void* q, const void* k, const void* v, const float* g, const float* beta,
                                   const int* chunk_start, const int* chunk_len, int NC, int H, int DK, float* G, void* w,
                                   void* u, void* qg, void* kg, void* Aqk, void* Ainv, void* Akk, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (DK == 128) return launch_fwd_intra<128>(q, k, v, g, beta, chunk_start, chunk_len, NC, H, G, w, u, qg, kg, Aqk, Ainv, Akk, s);
  if (DK == 64) return launch_fwd_intra<64>(q, k, v, g, beta, chunk_start, chunk_len, NC, H, G, w, u, qg, kg, Aqk, Ainv, Akk, s);
  return -1;
}

// ---------------------------------------------------------------------------------------------------
// Chunk table built on the device (no host sync): chunks never straddle a sequence boundary.
// cu: [N+1] int32. Outputs padded to nc_max entries; unused chunks get len 0.
__global__ void kda_build_chunks_kernel(const int* __restrict__ cu, int N, int* __restrict__ chunk_start,
                                        int* __restrict__ chunk_len, int* __restrict__ seq_chunk,
                                        int* __restrict__ seq_order, int nc_max) {
  __shared__ int total;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int n = 0; n < N; ++n) { seq_chunk[n] = acc; acc += (cu[n + 1] - cu[n] + 63) / 64; }
    seq_chunk[N] = acc;
    total = acc;
  }
  __syncthreads();
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    int s = cu[n], e = cu[n + 1], c = seq_chunk[n];
    for (; s < e; s += 64, ++c)
      if (c < nc_max) { chunk_start[c] = s; chunk_len[c] = min(64, e - s); }
  }
  for (int c = total + threadIdx.x; c < nc_max; c += blockDim.x) { chunk_start[c] = 0; chunk_len[c] = 0; }
  // launch order of the sequential state kernels: longest sequence first, so the longest chain starts at time 0
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    const int len_n = cu[n + 1] - cu[n];
    int rank = 0;
    for (int m = 0; m < N; ++m) {
      const int len_m = cu[m + 1] - cu[m];
      rank += (len_m > len_n) || (len_m == len_n && m < n);
    }
    seq_order[rank] = n;
  }
}

extern "C" int hippo_kda_build_chunks(const int* cu, int N, int* chunk_start, int* chunk_len, int* seq_chunk,
                                      int* seq_order, int nc_max, void* stream) {
  kda_build_chunks_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(cu, N, chunk_start, chunk_len, seq_chunk, seq_order, nc_max);
  return (int)cudaGetLastError();
}
