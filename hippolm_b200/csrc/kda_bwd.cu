// Chunked Kimi-Delta-Attention backward (chunk = 64 tokens, K = V = DK in {64, 128}).
//
//  kda_bwd_state   reverse recurrence over the chunks of a sequence (one CTA per sequence, head and
//                  32-column slice of V): dv_new = Aqk^T do + kg dS;  dS <- e^Glast dS + qg^T do - w^T dv_new
//  kda_bwd_dqkw    per (chunk, head): dAqk = tril(do v_new^T), dqg = do S^T, dkg = v_new dS^T,
//                  dw = -dv_new S^T, and the elementwise terms of qg / kg / the state decay
//  kda_bwd_wy      per (chunk, head): backward of u = Ainv (beta v), w = Ainv (beta k e^G) and of the
//                  triangular inverse (dAkk = -strict_lower(Ainv^T dAinv Ainv^T))
//  kda_bwd_amat    per (chunk, head): backward of the decayed Gram matrices (same sub-chunk anchoring
//                  as the forward), reverse cumsum of dG -> dg, final dq / dk
// Replaces fla/ops/kda/chunk_bwd.py:42-599, chunk_intra.py:367-629, fla/ops/common/chunk_delta_h.py:350-663.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <mma.h>
#include <stdint.h>
#include "kda_common.cuh"
#include <stdlib.h>

namespace hippo {
using namespace nvcuda;

typedef wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> FragA;
typedef wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::col_major> FragAT;
typedef wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> FragB;
typedef wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> FragBT;
typedef wmma::fragment<wmma::accumulator, 16, 16, 16, float> FragC;

// =================================================================================================== state
// 256 threads, one CTA per SM; the tiles of the next (earlier) chunk stream into the second shared-memory buffer
// with cp.async during the math of the current one.
template <int DK, int VS>
__global__ void __launch_bounds__(256, 1)
kda_bwd_state_kernel(const bf16* __restrict__ w, const bf16* __restrict__ qg, const bf16* __restrict__ kg,
                     const bf16* __restrict__ Aqk, const float* __restrict__ G, const bf16* __restrict__ d_o,
                     const int* __restrict__ chunk_start, const int* __restrict__ chunk_len,
                     const int* __restrict__ seq_chunk, const int* __restrict__ seq_order, int H,
                     const float* __restrict__ dfinal, bf16* __restrict__ dvn_out, bf16* __restrict__ dS_out,
                     float* __restrict__ dh0) {
  constexpr int LD = DK + 8, LS = VS + 8, LF = VS + 4, NTHR = 256;
  constexpr int NV_BIG = 64 * (DK / 8) / NTHR, NV_AQ = 64 * 8 / NTHR;
  static_assert(64 * (VS / 8) <= NTHR && DK <= NTHR, "tile/thread mapping");
  extern __shared__ __align__(128) uint8_t smem[];
  float* dS = (float*)smem;                   // [DK][LF]
  float* stg = dS + DK * LF;                  // [64][LF]
  float* egl = stg + 64 * LF;                 // [DK]
  bf16* dSb = (bf16*)(egl + DK);              // [DK][LS]
  bf16* ndv = dSb + DK * LS;                  // [64][LS]  (-dv_new)
  bf16* tiles = ndv + 64 * LS;                // 2 x { w, qg, kg: [64][LD] ; Aqk: [64][72] ; do: [64][LS] ; Glast: DK floats }
  constexpr int TILE_ELEMS = 3 * 64 * LD + 64 * 72 + 64 * LS + 2 * DK;

  const int vs0 = blockIdx.x * VS, h = blockIdx.y, seq = seq_order[blockIdx.z];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c_begin = seq_chunk[seq], c_end = seq_chunk[seq + 1];

  for (int idx = tid; idx < DK * VS; idx += NTHR) {
    int r = idx / VS, c = idx % VS;
    float s0 = dfinal ? dfinal[(((long long)seq * H + h) * DK + r) * DK + vs0 + c] : 0.f;
    dS[r * LF + c] = s0;
    dSb[r * LS + c] = __float2bfloat16(s0);
  }
  auto fetch = [&](int chunk, int buf) {
    const long long cbase = ((long long)chunk * H + h) * 64;
    const int t0 = chunk_start[chunk], len = chunk_len[chunk];
    bf16* tb = tiles + buf * TILE_ELEMS;
    bf16* ws_ = tb; bf16* qgs_ = ws_ + 64 * LD; bf16* kgs_ = qgs_ + 64 * LD; bf16* Aq_ = kgs_ + 64 * LD;
    bf16* dos_ = Aq_ + 64 * 72; float* gl_ = (float*)(dos_ + 64 * LS);
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
      const bool ok = r < len;                               // rows past the chunk end read as zeros
      cp_async16(dos_ + r * LS + c8, d_o + ((long long)(t0 + (ok ? r : 0)) * H + h) * DK + vs0 + c8, ok ? 16 : 0);
    }
    if (tid < DK / 4) cp_async16(gl_ + tid * 4, G + (cbase + 63) * DK + tid * 4);
    cp_async_commit();
  };
  if (c_begin < c_end) fetch(c_end - 1, 0);
  __syncthreads();

  for (int chunk = c_end - 1; chunk >= c_begin; --chunk) {
    const long long cbase = ((long long)chunk * H + h) * 64;
    const int buf = (c_end - 1 - chunk) & 1;
    bf16* ws = tiles + buf * TILE_ELEMS; bf16* qgs = ws + 64 * LD; bf16* kgs = qgs + 64 * LD; bf16* Aq = kgs + 64 * LD;
    bf16* dos = Aq + 64 * 72; const float* gl = (const float*)(dos + 64 * LS);
    cp_async_wait_all();
    __syncthreads();                                        // this chunk's tiles have landed; the other buffer is free
    if (chunk - 1 >= c_begin) fetch(chunk - 1, buf ^ 1);
    if (tid < DK) egl[tid] = __expf(gl[tid]);
    // gradient wrt the state after this chunk, for the per-chunk kernels
    for (int idx = tid; idx < DK * (VS / 8); idx += NTHR) {
      int r = idx / (VS / 8), c8 = (idx % (VS / 8)) * 8;
      *(uint4*)(dS_out + (((long long)chunk * H + h) * DK + r) * DK + vs0 + c8) = *(const uint4*)(dSb + r * LS + c8);
    }
    __syncthreads();
    // dv_new = Aqk^T do + kg dS
    const int rt = warp % 4, nt0 = warp / 4;
    {
      FragC acc; wmma::fill_fragment(acc, 0.f);
      for (int kt = rt; kt < 4; ++kt) {           // Aqk lower triangular -> Aqk^T upper
        FragAT a; FragB b;
        wmma::load_matrix_sync(a, Aq + kt * 16 * 72 + rt * 16, 72);
        wmma::load_matrix_sync(b, dos + kt * 16 * LS + nt0 * 16, LS);
        wmma::mma_sync(acc, a, b, acc);
      }
#pragma unroll
      for (int kt = 0; kt < DK / 16; ++kt) {
        FragA a; FragB b;
        wmma::load_matrix_sync(a, kgs + rt * 16 * LD + kt * 16, LD);
        wmma::load_matrix_sync(b, dSb + kt * 16 * LS + nt0 * 16, LS);
        wmma::mma_sync(acc, a, b, acc);
      }
      wmma::store_matrix_sync(stg + rt * 16 * LF + nt0 * 16, acc, LF, wmma::mem_row_major);
      __syncwarp();
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int el = lane * 8 + e, rr = rt * 16 + (el >> 4), cc = nt0 * 16 + (el & 15);
        float dv = stg[rr * LF + cc];
        dvn_out[(cbase + rr) * DK + vs0 + cc] = __float2bfloat16(dv);
        ndv[rr * LS + cc] = __float2bfloat16(-dv);
      }
    }
    __syncthreads();                              // ndv complete, dSb no longer read
    // dS <- e^Glast dS + qg^T do - w^T dv_new   (each warp owns its tiles)
    for (int t = warp; t < (DK / 16) * (VS / 16); t += 8) {
      const int mt = t / (VS / 16), nt = t % (VS / 16);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int el = lane * 8 + e, rr = mt * 16 + (el >> 4), cc = nt * 16 + (el & 15);
        dS[rr * LF + cc] *= egl[rr];
      }
      __syncwarp();
      FragC acc;
      wmma::load_matrix_sync(acc, dS + mt * 16 * LF + nt * 16, LF, wmma::mem_row_major);
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
        FragAT a; FragB b;
        wmma::load_matrix_sync(a, qgs + kt * 16 * LD + mt * 16, LD);
        wmma::load_matrix_sync(b, dos + kt * 16 * LS + nt * 16, LS);
        wmma::mma_sync(acc, a, b, acc);
        wmma::load_matrix_sync(a, ws + kt * 16 * LD + mt * 16, LD);
        wmma::load_matrix_sync(b, ndv + kt * 16 * LS + nt * 16, LS);
        wmma::mma_sync(acc, a, b, acc);
      }
      wmma::store_matrix_sync(dS + mt * 16 * LF + nt * 16, acc, LF, wmma::mem_row_major);
      __syncwarp();
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int el = lane * 8 + e, rr = mt * 16 + (el >> 4), cc = nt * 16 + (el & 15);
        dSb[rr * LS + cc] = __float2bfloat16(dS[rr * LF + cc]);
      }
    }
    __syncthreads();
  }
  if (dh0) {
    for (int idx = tid; idx < DK * VS; idx += NTHR) {
      int r = idx / VS, c = idx % VS;
      dh0[(((long long)seq * H + h) * DK + r) * DK + vs0 + c] = dS[r * LF + c];
    }
  }
}
template <int DK, int VS>
constexpr int kda_bwd_state_smem() {
  return DK * (VS + 4) * 4 + 64 * (VS + 4) * 4 + DK * 4 + DK * (VS + 8) * 2 + 64 * (VS + 8) * 2 +
         2 * (3 * 64 * (DK + 8) + 64 * 72 + 64 * (VS + 8) + 2 * DK) * 2 + 128;
}

// Register-resident variant for DK = 128 (mma.sync m16n8k16 + ldmatrix): warp w keeps rows 16w..16w+15 of the fp32
// state gradient in registers across the whole (reverse) chain; only its bf16 image lives in shared memory as the B
// operand of the next chunk. Two barriers per chunk, tiles double-buffered with cp.async.
template <int VS>
__global__ void __launch_bounds__(256, 1)
kda_bwd_state_mma_kernel(const bf16* __restrict__ w, const bf16* __restrict__ qg, const bf16* __restrict__ kg,
                         const bf16* __restrict__ Aqk, const float* __restrict__ G, const bf16* __restrict__ d_o,
                         const int* __restrict__ chunk_start, const int* __restrict__ chunk_len,
                         const int* __restrict__ seq_chunk, const int* __restrict__ seq_order, int H,
                         const float* __restrict__ dfinal, bf16* __restrict__ dvn_out, bf16* __restrict__ dS_out,
                         float* __restrict__ dh0) {
  constexpr int DK = 128, LD = DK + 8, LS = VS + 8, LQ = 72, NTHR = 256;
  static_assert(VS == 32, "warp tiling below assumes a 32-column value slice");
  constexpr int TILE_ELEMS = 3 * 64 * LD + 64 * LQ + 64 * LS + 2 * DK;
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* tiles = (bf16*)smem;                                 // 2 x { w, qg, kg: [64][LD]; Aqk: [64][LQ]; do: [64][LS]; Glast }
  bf16* dSb = tiles + 2 * TILE_ELEMS;                        // [DK][LS]
  bf16* ndv = dSb + DK * LS;                                 // [64][LS]   (-dv_new)
  float* egl = (float*)(ndv + 64 * LS);                      // [DK]

  const int vs0 = blockIdx.x * VS, h = blockIdx.y, seq = seq_order[blockIdx.z];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int c_begin = seq_chunk[seq], c_end = seq_chunk[seq + 1];
  if (c_begin >= c_end) return;
  const int mt = warp & 3, nh = warp >> 2;
  const int srow = warp * 16 + g;

  float dS[4][4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const int c = vs0 + nt * 8 + 2 * t4;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = srow + (e >> 1) * 8;
      dS[nt][e] = dfinal ? dfinal[(((long long)seq * H + h) * DK + r) * DK + c + (e & 1)] : 0.f;
    }
    *(unsigned*)(dSb + srow * LS + nt * 8 + 2 * t4) = kda_pack2(dS[nt][0], dS[nt][1]);
    *(unsigned*)(dSb + (srow + 8) * LS + nt * 8 + 2 * t4) = kda_pack2(dS[nt][2], dS[nt][3]);
  }
  auto fetch = [&](int chunk, int buf) {
    const long long cbase = ((long long)chunk * H + h) * 64;
    const int t0 = chunk_start[chunk], len = chunk_len[chunk];
    bf16* ws_ = tiles + buf * TILE_ELEMS; bf16* qgs_ = ws_ + 64 * LD; bf16* kgs_ = qgs_ + 64 * LD; bf16* Aq_ = kgs_ + 64 * LD;
    bf16* dos_ = Aq_ + 64 * LQ; float* gl_ = (float*)(dos_ + 64 * LS);
#pragma unroll
    for (int j = 0; j < 64 * (DK / 8) / NTHR; ++j) {
      const int idx = tid + j * NTHR, r = idx >> 4, c8 = (idx & 15) * 8;
      const long long off = (cbase + r) * DK + c8;
      cp_async16(ws_ + r * LD + c8, w + off); cp_async16(qgs_ + r * LD + c8, qg + off); cp_async16(kgs_ + r * LD + c8, kg + off);
    }
#pragma unroll
    for (int j = 0; j < 64 * 8 / NTHR; ++j) {
      const int idx = tid + j * NTHR, r = idx >> 3, c8 = (idx & 7) * 8;
      cp_async16(Aq_ + r * LQ + c8, Aqk + (cbase + r) * 64 + c8);
    }
    {
      const int r = tid >> 2, c8 = (tid & 3) * 8;
      const bool ok = r < len;                               // rows past the chunk end read as zeros
      cp_async16(dos_ + r * LS + c8, d_o + ((long long)(t0 + (ok ? r : 0)) * H + h) * DK + vs0 + c8, ok ? 16 : 0);
    }
    if (tid < DK / 4) cp_async16(gl_ + tid * 4, G + (cbase + 63) * DK + tid * 4);
    cp_async_commit();
  };
  fetch(c_end - 1, 0);
  cp_async_wait_all();
  __syncthreads();

  for (int chunk = c_end - 1; chunk >= c_begin; --chunk) {
    const long long cbase = ((long long)chunk * H + h) * 64;
    const int buf = (c_end - 1 - chunk) & 1;
    const bf16* ws = tiles + buf * TILE_ELEMS; const bf16* qgs = ws + 64 * LD; const bf16* kgs = qgs + 64 * LD;
    const bf16* Aq = kgs + 64 * LD; const bf16* dos = Aq + 64 * LQ; const float* gl = (const float*)(dos + 64 * LS);
    if (chunk - 1 >= c_begin) fetch(chunk - 1, buf ^ 1);     // the other buffer was released at the last barrier
    if (tid < DK) egl[tid] = __expf(gl[tid]);
    // gradient wrt the state after this chunk, for the per-chunk kernels
#pragma unroll
    for (int j = 0; j < DK * (VS / 8) / NTHR; ++j) {
      const int idx = tid + j * NTHR, r = idx / (VS / 8), c8 = (idx % (VS / 8)) * 8;
      *(uint4*)(dS_out + (((long long)chunk * H + h) * DK + r) * DK + vs0 + c8) = *(const uint4*)(dSb + r * LS + c8);
    }
    // ---- dv_new = Aqk^T do + kg dS   (rows mt*16.., columns nh*16..)
    {
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      for (int kt = mt; kt < 4; ++kt) {                      // Aqk lower triangular -> Aqk^T upper
        unsigned af[4], b[4];
        kda_frag_a_t(af, Aq, LQ, mt * 16, kt * 16, lane);
        kda_frag_b2(b, dos, LS, kt * 16, nh * 16, lane);
        kda_mma16816(acc[0], af, b[0], b[1]);
        kda_mma16816(acc[1], af, b[2], b[3]);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        unsigned af[4], b[4];
        kda_frag_a(af, kgs, LD, mt * 16, kk * 16, lane);
        kda_frag_b2(b, dSb, LS, kk * 16, nh * 16, lane);
        kda_mma16816(acc[0], af, b[0], b[1]);
        kda_mma16816(acc[1], af, b[2], b[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const int c = nh * 16 + nt * 8 + 2 * t4;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = mt * 16 + g + hh * 8;
          *(unsigned*)(dvn_out + (cbase + r) * DK + vs0 + c) = kda_pack2(acc[nt][2 * hh], acc[nt][2 * hh + 1]);
          *(unsigned*)(ndv + r * LS + c) = kda_pack2(-acc[nt][2 * hh], -acc[nt][2 * hh + 1]);
        }
      }
    }
    __syncthreads();                                          // ndv complete; every warp is past its reads of dSb
    // ---- dS <- e^Glast dS + qg^T do - w^T dv_new   (this warp's 16 rows, all VS columns)
    {
      const float e0 = egl[srow], e1 = egl[srow + 8];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) { dS[nt][0] *= e0; dS[nt][1] *= e0; dS[nt][2] *= e1; dS[nt][3] *= e1; }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        unsigned af[4], b0[4], b1[4];
        kda_frag_a_t(af, qgs, LD, warp * 16, kk * 16, lane);
        kda_frag_b2(b0, dos, LS, kk * 16, 0, lane);
        kda_frag_b2(b1, dos, LS, kk * 16, 16, lane);
        kda_mma16816(dS[0], af, b0[0], b0[1]);
        kda_mma16816(dS[1], af, b0[2], b0[3]);
        kda_mma16816(dS[2], af, b1[0], b1[1]);
        kda_mma16816(dS[3], af, b1[2], b1[3]);
        kda_frag_a_t(af, ws, LD, warp * 16, kk * 16, lane);
        kda_frag_b2(b0, ndv, LS, kk * 16, 0, lane);
        kda_frag_b2(b1, ndv, LS, kk * 16, 16, lane);
        kda_mma16816(dS[0], af, b0[0], b0[1]);
        kda_mma16816(dS[1], af, b0[2], b0[3]);
        kda_mma16816(dS[2], af, b1[0], b1[1]);
        kda_mma16816(dS[3], af, b1[2], b1[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        *(unsigned*)(dSb + srow * LS + nt * 8 + 2 * t4) = kda_pack2(dS[nt][0], dS[nt][1]);
        *(unsigned*)(dSb + (srow + 8) * LS + nt * 8 + 2 * t4) = kda_pack2(dS[nt][2], dS[nt][3]);
      }
    }
    cp_async_wait_all();                                      // the next (earlier) chunk's tiles have landed
    __syncthreads();
  }
  if (dh0) {
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int c = vs0 + nt * 8 + 2 * t4;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        *(float2*)(dh0 + (((long long)seq * H + h) * DK + srow + hh * 8) * DK + c) = make_float2(dS[nt][2 * hh], dS[nt][2 * hh + 1]);
    }
  }
}
template <int VS>
constexpr int kda_bwd_state_mma_smem() {
  return (2 * (3 * 64 * 136 + 64 * 72 + 64 * (VS + 8) + 2 * 128) + 128 * (VS + 8) + 64 * (VS + 8)) * 2 + 128 * 4 + 128;
}

// =================================================================================================== dqkw
template <int DK>
__global__ void __launch_bounds__(512, 1)
kda_bwd_dqkw_kernel(const bf16* __restrict__ d_o, const bf16* __restrict__ vnew, const bf16* __restrict__ dvn,
                    const bf16* __restrict__ Sst, const bf16* __restrict__ dSst, const bf16* __restrict__ qg,
                    const bf16* __restrict__ kg, const float* __restrict__ G, const int* __restrict__ chunk_start,
                    const int* __restrict__ chunk_len, int H, float* __restrict__ dq_acc, float* __restrict__ dk_acc,
                    float* __restrict__ dG_acc, bf16* __restrict__ dw_out, bf16* __restrict__ dAqk_out) {
  constexpr int LD = DK + 8, NT = DK / 16;
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* dos = (bf16*)smem;            // [64][LD]
  bf16* vns = dos + 64 * LD;
  bf16* dvs = vns + 64 * LD;
  bf16* Ss = dvs + 64 * LD;           // [DK][LD]
  bf16* dSs = Ss + DK * LD;           // [DK][LD]
  float* stg = (float*)(dSs + DK * LD);   // [16 warps][2][16][20]
  float* dGl = stg + 16 * 2 * 320;    // [DK]
  const int chunk = blockIdx.x, h = blockIdx.y;
  const int t0 = chunk_start[chunk], len = chunk_len[chunk];
  if (len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long cbase = ((long long)chunk * H + h) * 64;
  const long long sbase = ((long long)chunk * H + h) * DK;

  for (int idx = tid; idx < 64 * (DK / 8); idx += 512) {
    int r = idx / (DK / 8), c8 = (idx % (DK / 8)) * 8;
    uint4 z = make_uint4(0, 0, 0, 0);
    if (r < len) z = *(const uint4*)(d_o + ((long long)(t0 + r) * H + h) * DK + c8);
    *(uint4*)(dos + r * LD + c8) = z;
    *(uint4*)(vns + r * LD + c8) = *(const uint4*)(vnew + (cbase + r) * DK + c8);
    *(uint4*)(dvs + r * LD + c8) = *(const uint4*)(dvn + (cbase + r) * DK + c8);
  }
  for (int idx = tid; idx < DK * (DK / 8); idx += 512) {
    int r = idx / (DK / 8), c8 = (idx % (DK / 8)) * 8;
    *(uint4*)(Ss + r * LD + c8) = *(const uint4*)(Sst + (sbase + r) * DK + c8);
    *(uint4*)(dSs + r * LD + c8) = *(const uint4*)(dSst + (sbase + r) * DK + c8);
  }
  if (tid < DK) dGl[tid] = 0.f;
  __syncthreads();
  // state-decay term of dGlast: sum_v dS[c,v] S[c,v] e^Glast[c]
  {
    constexpr int TPR = 512 / DK;           // threads per state row
    int c = tid / TPR, part = tid % TPR;
    float s = 0.f;
    for (int vv = part; vv < DK; vv += TPR)
      s += __bfloat162float(Ss[c * LD + vv]) * __bfloat162float(dSs[c * LD + vv]);
    s *= __expf(G[(cbase + 63) * DK + c]);
    atomicAdd(&dGl[c], s);
  }
  float* my0 = stg + warp * 640, *my1 = my0 + 320;
  // (dqg, dkg) pairs: one warp does both for a given 16x16 tile so that dG has a single writer
  for (int t = warp; t < 4 * NT; t += 16) {
    const int rt = t / NT, nt = t % NT;
    FragC a0, a1; wmma::fill_fragment(a0, 0.f); wmma::fill_fragment(a1, 0.f);
#pragma unroll
    for (int kt = 0; kt < NT; ++kt) {
      FragA a; FragBT b;
      wmma::load_matrix_sync(a, dos + rt * 16 * LD + kt * 16, LD);
      wmma::load_matrix_sync(b, Ss + nt * 16 * LD + kt * 16, LD);       // S^T
      wmma::mma_sync(a0, a, b, a0);
      wmma::load_matrix_sync(a, vns + rt * 16 * LD + kt * 16, LD);
      wmma::load_matrix_sync(b, dSs + nt * 16 * LD + kt * 16, LD);      // dS^T
      wmma::mma_sync(a1, a, b, a1);
    }
    wmma::store_matrix_sync(my0, a0, 20, wmma::mem_row_major);
    wmma::store_matrix_sync(my1, a1, 20, wmma::mem_row_major);
    __syncwarp();
    // lane -> column cc = lane & 15, rows rr = (lane >> 4) * 8 .. +7
    {
      const int cc = lane & 15, rbase = (lane >> 4) * 8, c = nt * 16 + cc;
      const float gl = G[(cbase + 63) * DK + c];
      float colsum = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int rr = rbase + e, i = rt * 16 + rr;
        const long long off = (cbase + i) * DK + c;
        const float Gi = G[off];
        const float dqgv = my0[rr * 20 + cc], dkgv = my1[rr * 20 + cc];
        const float qgv = __bfloat162float(qg[off]), kgv = __bfloat162float(kg[off]);
        dq_acc[off] = dqgv * __expf(Gi);
        dk_acc[off] = dkgv * __expf(gl - Gi);
        dG_acc[off] = dqgv * qgv - dkgv * kgv;
        colsum += dkgv * kgv;
      }
      colsum += __shfl_xor_sync(0xFFFFFFFFu, colsum, 16);
      if (lane < 16) atomicAdd(&dGl[c], colsum);
    }
    __syncwarp();
  }
  // dw = -dv_new S^T
  for (int t = warp; t < 4 * NT; t += 16) {
    const int rt = t / NT, nt = t % NT;
    FragC a0; wmma::fill_fragment(a0, 0.f);
#pragma unroll
    for (int kt = 0; kt < NT; ++kt) {
      FragA a; FragBT b;
      wmma::load_matrix_sync(a, dvs + rt * 16 * LD + kt * 16, LD);
      wmma::load_matrix_sync(b, Ss + nt * 16 * LD + kt * 16, LD);
      wmma::mma_sync(a0, a, b, a0);
    }
    wmma::store_matrix_sync(my0, a0, 20, wmma::mem_row_major);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      int el = lane * 8 + e, rr = el >> 4, cc = el & 15;
      dw_out[(cbase + rt * 16 + rr) * DK + nt * 16 + cc] = __float2bfloat16(-my0[rr * 20 + cc]);
    }
    __syncwarp();
  }
  // dAqk = tril(do v_new^T)
  for (int t = warp; t < 16; t += 16) {
    const int rt = t >> 2, ct = t & 3;
    FragC a0; wmma::fill_fragment(a0, 0.f);
    if (ct <= rt) {
#pragma unroll
      for (int kt = 0; kt < NT; ++kt) {
        FragA a; FragBT b;
        wmma::load_matrix_sync(a, dos + rt * 16 * LD + kt * 16, LD);
        wmma::load_matrix_sync(b, vns + ct * 16 * LD + kt * 16, LD);    // v_new^T
        wmma::mma_sync(a0, a, b, a0);
      }
    }
    wmma::store_matrix_sync(my0, a0, 20, wmma::mem_row_major);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      int el = lane * 8 + e, rr = el >> 4, cc = el & 15;
      int i = rt * 16 + rr, j = ct * 16 + cc;
      dAqk_out[(cbase + i) * 64 + j] = __float2bfloat16(j <= i ? my0[rr * 20 + cc] : 0.f);
    }
    __syncwarp();
  }
  __syncthreads();
  if (tid < DK) dG_acc[(cbase + 63) * DK + tid] += dGl[tid];
}
template <int DK>
constexpr int kda_bwd_dqkw_smem() { return 3 * 64 * (DK + 8) * 2 + 2 * DK * (DK + 8) * 2 + 16 * 2 * 320 * 4 + DK * 4 + 128; }

// mma.sync variant for DK = 128: the four products of a chunk share one K loop (A fragments of do / v_new / dv_new,
// B fragments of S^T and dS^T loaded once per step) and the epilogue works on the accumulator fragments directly.
// 16 warps: warp (rt, ng) owns rows rt*16.. and columns ng*32.. of dqg / dkg / dw, and tile (rt, ct = ng) of dAqk.
__global__ void __launch_bounds__(512, 1)
kda_bwd_dqkw_mma_kernel(const bf16* __restrict__ d_o, const bf16* __restrict__ vnew, const bf16* __restrict__ dvn,
                        const bf16* __restrict__ Sst, const bf16* __restrict__ dSst, const bf16* __restrict__ qg,
                        const bf16* __restrict__ kg, const float* __restrict__ G, const int* __restrict__ chunk_start,
                        const int* __restrict__ chunk_len, int H, float* __restrict__ dq_acc, float* __restrict__ dk_acc,
                        float* __restrict__ dG_acc, bf16* __restrict__ dw_out, bf16* __restrict__ dAqk_out) {
  constexpr int DK = 128, LD = DK + 8;
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* dos = (bf16*)smem;            // [64][LD]
  bf16* vns = dos + 64 * LD;
  bf16* dvs = vns + 64 * LD;
  bf16* Ss = dvs + 64 * LD;           // [DK][LD]   S[c][v]
  bf16* dSs = Ss + DK * LD;           // [DK][LD]
  float* dGl = (float*)(dSs + DK * LD);   // [DK]
  const int chunk = blockIdx.x, h = blockIdx.y;
  const int t0 = chunk_start[chunk], len = chunk_len[chunk];
  if (len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const long long cbase = ((long long)chunk * H + h) * 64;
  const long long sbase = ((long long)chunk * H + h) * DK;

  for (int idx = tid; idx < 64 * (DK / 8); idx += 512) {
    const int r = idx >> 4, c8 = (idx & 15) * 8;
    cp_async16(dos + r * LD + c8, d_o + ((long long)(t0 + (r < len ? r : 0)) * H + h) * DK + c8, r < len ? 16 : 0);
    cp_async16(vns + r * LD + c8, vnew + (cbase + r) * DK + c8);
    cp_async16(dvs + r * LD + c8, dvn + (cbase + r) * DK + c8);
  }
  for (int idx = tid; idx < DK * (DK / 8); idx += 512) {
    const int r = idx >> 4, c8 = (idx & 15) * 8;
    cp_async16(Ss + r * LD + c8, Sst + (sbase + r) * DK + c8);
    cp_async16(dSs + r * LD + c8, dSst + (sbase + r) * DK + c8);
  }
  cp_async_commit();
  if (tid < DK) dGl[tid] = 0.f;
  cp_async_wait_all();
  __syncthreads();
  // state-decay term of dGlast: sum_v dS[c,v] S[c,v] e^Glast[c]   (4 threads per state row)
  {
    const int c = tid >> 2, part = tid & 3;
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 a = *(const uint4*)(Ss + c * LD + part * 32 + j * 8), b = *(const uint4*)(dSs + c * LD + part * 32 + j * 8);
      const __nv_bfloat162* ab = (const __nv_bfloat162*)&a; const __nv_bfloat162* bb = (const __nv_bfloat162*)&b;
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float2 x = __bfloat1622float2(ab[e]), y = __bfloat1622float2(bb[e]); s += x.x * y.x + x.y * y.y; }
    }
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
    if (part == 0) atomicAdd(&dGl[c], s * __expf(G[(cbase + 63) * DK + c]));
  }
  const int rt = warp & 3, ng = warp >> 2;
  float aq[4][4], ak[4][4], aw[4][4], aa[2][4];
#pragma unroll
  for (int n = 0; n < 4; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) { aq[n][e] = 0.f; ak[n][e] = 0.f; aw[n][e] = 0.f; }
#pragma unroll
  for (int n = 0; n < 2; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) aa[n][e] = 0.f;
  const bool do_a = ng <= rt;                        // lower-triangular 16x16 tiles of dAqk
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    unsigned fo[4], fv[4], fd[4], b0[4], b1[4];
    kda_frag_a(fo, dos, LD, rt * 16, kk * 16, lane);
    kda_frag_a(fv, vns, LD, rt * 16, kk * 16, lane);
    kda_frag_a(fd, dvs, LD, rt * 16, kk * 16, lane);
    kda_frag_bt2(b0, Ss, LD, ng * 32, kk * 16, lane);        // S^T: n = state row c, k = v
    kda_frag_bt2(b1, Ss, LD, ng * 32 + 16, kk * 16, lane);
    kda_mma16816(aq[0], fo, b0[0], b0[1]); kda_mma16816(aq[1], fo, b0[2], b0[3]);
    kda_mma16816(aq[2], fo, b1[0], b1[1]); kda_mma16816(aq[3], fo, b1[2], b1[3]);
    kda_mma16816(aw[0], fd, b0[0], b0[1]); kda_mma16816(aw[1], fd, b0[2], b0[3]);
    kda_mma16816(aw[2], fd, b1[0], b1[1]); kda_mma16816(aw[3], fd, b1[2], b1[3]);
    kda_frag_bt2(b0, dSs, LD, ng * 32, kk * 16, lane);
    kda_frag_bt2(b1, dSs, LD, ng * 32 + 16, kk * 16, lane);
    kda_mma16816(ak[0], fv, b0[0], b0[1]); kda_mma16816(ak[1], fv, b0[2], b0[3]);
    kda_mma16816(ak[2], fv, b1[0], b1[1]); kda_mma16816(ak[3], fv, b1[2], b1[3]);
    if (do_a) {
      kda_frag_bt2(b0, vns, LD, ng * 16, kk * 16, lane);     // v_new^T: n = chunk row j, k = v
      kda_mma16816(aa[0], fo, b0[0], b0[1]); kda_mma16816(aa[1], fo, b0[2], b0[3]);
    }
  }
  // ---- epilogue on the fragments: thread holds rows i0, i0+8 and column pairs c, c+1 of each n-tile
  const int i0 = rt * 16 + g;
#pragma unroll
  for (int n = 0; n < 4; ++n) {
    const int c = ng * 32 + n * 8 + 2 * t4;
    const float2 gl = *(const float2*)(G + (cbase + 63) * DK + c);
    float cs0 = 0.f, cs1 = 0.f;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const long long off = (cbase + i0 + hh * 8) * DK + c;
      const float2 Gi = *(const float2*)(G + off);
      const float2 qv = __bfloat1622float2(*(const __nv_bfloat162*)(qg + off));
      const float2 kv = __bfloat1622float2(*(const __nv_bfloat162*)(kg + off));
      const float dq0 = aq[n][2 * hh], dq1 = aq[n][2 * hh + 1], dk0 = ak[n][2 * hh], dk1 = ak[n][2 * hh + 1];
      *(float2*)(dq_acc + off) = make_float2(dq0 * __expf(Gi.x), dq1 * __expf(Gi.y));
      *(float2*)(dk_acc + off) = make_float2(dk0 * __expf(gl.x - Gi.x), dk1 * __expf(gl.y - Gi.y));
      *(float2*)(dG_acc + off) = make_float2(dq0 * qv.x - dk0 * kv.x, dq1 * qv.y - dk1 * kv.y);
      cs0 += dk0 * kv.x; cs1 += dk1 * kv.y;
      *(unsigned*)(dw_out + off) = kda_pack2(-aw[n][2 * hh], -aw[n][2 * hh + 1]);
    }
    // column sums over the 16 rows of this tile: lanes with the same t4
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) { cs0 += __shfl_xor_sync(0xFFFFFFFFu, cs0, o); cs1 += __shfl_xor_sync(0xFFFFFFFFu, cs1, o); }
    if (g == 0) { atomicAdd(&dGl[c], cs0); atomicAdd(&dGl[c + 1], cs1); }
  }
  // dAqk = tril(do v_new^T): warp (rt, ct = ng) writes its 16x16 tile, zeros above the diagonal
#pragma unroll
  for (int n = 0; n < 2; ++n) {
    const int j = ng * 16 + n * 8 + 2 * t4;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int i = i0 + hh * 8;
      const float v0 = (do_a && j <= i) ? aa[n][2 * hh] : 0.f, v1 = (do_a && j + 1 <= i) ? aa[n][2 * hh + 1] : 0.f;
      *(unsigned*)(dAqk_out + (cbase + i) * 64 + j) = kda_pack2(v0, v1);
    }
  }
  __syncthreads();
  // the element (63, c) of dG_acc was written above by the warp owning row 63; its writer is inside this CTA
  if (tid < DK) dG_acc[(cbase + 63) * DK + tid] += dGl[tid];
}
constexpr int kda_bwd_dqkw_mma_smem() { return 3 * 64 * 136 * 2 + 2 * 128 * 136 * 2 + 128 * 4 + 128; }

// =================================================================================================== WY
template <int DK>
__global__ void __launch_bounds__(256, 2)
kda_bwd_wy_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, const float* __restrict__ beta,
                  const float* __restrict__ G, const bf16* __restrict__ Ainv, const bf16* __restrict__ Akk,
                  const bf16* __restrict__ dvn, const bf16* __restrict__ dw, const int* __restrict__ chunk_start,
                  const int* __restrict__ chunk_len, int H, bf16* __restrict__ dbk_out,
                  bf16* __restrict__ dv_out, float* __restrict__ dbeta_out, bf16* __restrict__ dKK_out) {
  constexpr int LD = DK + 8, NT = DK / 16;
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* Xb = (bf16*)smem;             // [64][72]
  bf16* dXb = Xb + 64 * 72;           // [64][72]
  bf16* Yb = dXb + 64 * 72;           // [64][72]
  bf16* dus = Yb + 64 * 72;           // [64][LD]
  bf16* dws = dus + 64 * LD;
  bf16* bks = dws + 64 * LD;          // beta k e^G
  bf16* bvs = bks + 64 * LD;          // beta v
  float* stg = (float*)(bvs + 64 * LD);   // [8][16][20]
  float* bs = stg + 8 * 320;          // [64]
  float* dbs = bs + 64;               // [64]
  const int chunk = blockIdx.x, h = blockIdx.y;
  const int t0 = chunk_start[chunk], len = chunk_len[chunk];
  if (len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long cbase = ((long long)chunk * H + h) * 64;

  if (tid < 64) { bs[tid] = tid < len ? beta[(long long)(t0 + tid) * H + h] : 0.f; dbs[tid] = 0.f; }
  for (int idx = tid; idx < 64 * 8; idx += 256) {
    int r = idx >> 3, c8 = (idx & 7) * 8;
    *(uint4*)(Xb + r * 72 + c8) = *(const uint4*)(Ainv + (cbase + r) * 64 + c8);
  }
  for (int idx = tid; idx < 64 * (DK / 8); idx += 256) {
    int r = idx / (DK / 8), c8 = (idx % (DK / 8)) * 8;
    *(uint4*)(dus + r * LD + c8) = *(const uint4*)(dvn + (cbase + r) * DK + c8);
    *(uint4*)(dws + r * LD + c8) = *(const uint4*)(dw + (cbase + r) * DK + c8);
  }
  __syncthreads();
  for (int idx = tid; idx < 64 * DK; idx += 256) {
    int i = idx / DK, c = idx % DK;
    float kv = 0.f, vv = 0.f;
    if (i < len) {
      long long off = ((long long)(t0 + i) * H + h) * DK + c;
      kv = __bfloat162float(k[off]); vv = __bfloat162float(v[off]);
    }
    bks[i * LD + c] = __float2bfloat16(bs[i] * kv * __expf(G[(cbase + i) * DK + c]));
    bvs[i * LD + c] = __float2bfloat16(bs[i] * vv);
  }
  __syncthreads();
  float* my = stg + warp * 320;
  // dX = du bv^T + dw bk^T  (only the lower triangle feeds dAkk)
  for (int t = warp; t < 16; t += 8) {
    const int rt = t >> 2, ct = t & 3;
    FragC acc; wmma::fill_fragment(acc, 0.f);
    if (ct <= rt) {
#pragma unroll
      for (int kt = 0; kt < NT; ++kt) {
        FragA a; FragBT b;
        wmma::load_matrix_sync(a, dus + rt * 16 * LD + kt * 16, LD);
        wmma::load_matrix_sync(b, bvs + ct * 16 * LD + kt * 16, LD);
        wmma::mma_sync(acc, a, b, acc);
        wmma::load_matrix_sync(a, dws + rt * 16 * LD + kt * 16, LD);
        wmma::load_matrix_sync(b, bks + ct * 16 * LD + kt * 16, LD);
        wmma::mma_sync(acc, a, b, acc);
      }
    }
    wmma::store_matrix_sync(my, acc, 20, wmma::mem_row_major);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      int el = lane * 8 + e, rr = el >> 4, cc = el & 15;
      dXb[(rt * 16 + rr) * 72 + ct * 16 + cc] = __float2bfloat16(my[rr * 20 + cc]);
    }
    __syncwarp();
  }
  __syncthreads();
  // Y = X^T dX
  for (int t = warp; t < 16; t += 8) {
    const int rt = t >> 2, ct = t & 3;
    FragC acc; wmma::fill_fragment(acc, 0.f);
    for (int kt = rt; kt < 4; ++kt) {            // X^T[i,m] = X[m,i], non-zero for m >= i
      FragAT a; FragB b;
      wmma::load_matrix_sync(a, Xb + kt * 16 * 72 + rt * 16, 72);
      wmma::load_matrix_sync(b, dXb + kt * 16 * 72 + ct * 16, 72);
      wmma::mma_sync(acc, a, b, acc);
    }
    wmma::store_matrix_sync(my, acc, 20, wmma::mem_row_major);
    __syncwarp();
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      int el = lane * 8 + e, rr = el >> 4, cc = el & 15;
      Yb[(rt * 16 + rr) * 72 + ct * 16 + cc] = __float2bfloat16(my[rr * 20 + cc]);
    }
    __syncwarp();
  }
  __syncthreads();
  // dM = -Y X^T ; dAkk = strict_lower(dM) ; dKK = beta_i dAkk ; dbeta_i += sum_j dAkk Akk / beta_i
  for (int t = warp; t < 16; t += 8) {
    const int rt = t >> 2, ct = t & 3;
    FragC acc; wmma::fill_fragment(acc, 0.f);
    if (ct <= rt) {
      for (int kt = 0; kt <= ct; ++kt) {         // X^T[n,j] = X[j,n], non-zero for n <= j
        FragA a; FragBT b;
        wmma::load_matrix_sync(a, Yb + rt * 16 * 72 + kt * 16, 72);
        wmma::load_matrix_sync(b, Xb + ct * 16 * 72 + kt * 16, 72);
        wmma::mma_sync(acc, a, b, acc);
      }
    }
    wmma::store_matrix_sync(my, acc, 20, wmma::mem_row_major);
    __syncwarp();
    {
      const int rr = lane >> 1, half = lane & 1, i = rt * 16 + rr;
      float rowsum = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        int cc = half * 8 + e, j = ct * 16 + cc;
        float dA = j < i ? -my[rr * 20 + cc] : 0.f;
        float a = __bfloat162float(Akk[(cbase + i) * 64 + j]);
        rowsum += dA * a;
        dKK_out[(cbase + i) * 64 + j] = __float2bfloat16(dA * bs[i]);
      }
      rowsum += __shfl_xor_sync(0xFFFFFFFFu, rowsum, 1);
      if (half == 0 && bs[i] > 0.f) atomicAdd(&dbs[i], rowsum / bs[i]);
    }
    __syncwarp();
  }
  // dbv = X^T du -> dv, dbeta ;  dbk = X^T dw -> dk, dG, dbeta
  for (int t = warp; t < 2 * 4 * NT; t += 8) {
    const int which = t / (4 * NT), rt = (t % (4 * NT)) / NT, nt = t % NT;
    const bf16* B = which ? dws : dus;
    FragC acc; wmma::fill_fragment(acc, 0.f);
    for (int kt = rt; kt < 4; ++kt) {
      FragAT a; FragB b;
      wmma::load_matrix_sync(a, Xb + kt * 16 * 72 + rt * 16, 72);
      wmma::load_matrix_sync(b, B + kt * 16 * LD + nt * 16, LD);
      wmma::mma_sync(acc, a, b, acc);
    }
    wmma::store_matrix_sync(my, acc, 20, wmma::mem_row_major);
    __syncwarp();
    {
      const int rr = lane >> 1, half = lane & 1, i = rt * 16 + rr;
      float rowsum = 0.f;
      if (!which) {
        // dv = beta * dbv ; dbeta += sum_c v * dbv  (v recovered from the beta*v tile)
        const float inv_b = bs[i] > 0.f ? 1.f / bs[i] : 0.f;
        float o8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int cc = half * 8 + e, c = nt * 16 + cc;
          const float val = my[rr * 20 + cc];
          o8[e] = bs[i] * val;
          rowsum += __bfloat162float(bvs[i * LD + c]) * inv_b * val;
        }
        if (i < len) {
          uint4 pk; __nv_bfloat162* pb = (__nv_bfloat162*)&pk;
#pragma unroll
          for (int e = 0; e < 4; ++e) pb[e] = __floats2bfloat162_rn(o8[2 * e], o8[2 * e + 1]);
          *(uint4*)(dv_out + ((long long)(t0 + i) * H + h) * DK + nt * 16 + half * 8) = pk;
        }
        rowsum += __shfl_xor_sync(0xFFFFFFFFu, rowsum, 1);
        if (half == 0 && i < len) atomicAdd(&dbs[i], rowsum);
      } else {
        // dbk = X^T dw is consumed by the A-matrix kernel (dk, dG and the k part of dbeta)
        uint4 pk; __nv_bfloat162* pb = (__nv_bfloat162*)&pk;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          pb[e] = __floats2bfloat162_rn(my[rr * 20 + half * 8 + 2 * e], my[rr * 20 + half * 8 + 2 * e + 1]);
        *(uint4*)(dbk_out + (cbase + i) * DK + nt * 16 + half * 8) = pk;
      }
    }
    __syncwarp();
  }
  __syncthreads();
  if (tid < len) dbeta_out[(long long)(t0 + tid) * H + h] = dbs[tid];
}
template <int DK>
constexpr int kda_bwd_wy_smem() { return 3 * 64 * 72 * 2 + 4 * 64 * (DK + 8) * 2 + 8 * 320 * 4 + 128 * 4 + 128; }

// mma.sync variant for DK = 128: every product works on accumulator fragments (no staging tile), the epilogues run on
// the fragments directly. 8 warps, two CTAs per SM.
__global__ void __launch_bounds__(256, 2)
kda_bwd_wy_mma_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, const float* __restrict__ beta,
                      const float* __restrict__ G, const bf16* __restrict__ Ainv, const bf16* __restrict__ Akk,
                      const bf16* __restrict__ dvn, const bf16* __restrict__ dw, const int* __restrict__ chunk_start,
                      const int* __restrict__ chunk_len, int H, bf16* __restrict__ dbk_out,
                      bf16* __restrict__ dv_out, float* __restrict__ dbeta_out, bf16* __restrict__ dKK_out) {
  constexpr int DK = 128, LD = DK + 8, LX = 72;
  extern __shared__ __align__(128) uint8_t smem[];
  bf16* Xb = (bf16*)smem;             // [64][LX]  X = (I + Akk)^-1
  bf16* dXb = Xb + 64 * LX;           // [64][LX]
  bf16* Yb = dXb + 64 * LX;           // [64][LX]
  bf16* dus = Yb + 64 * LX;           // [64][LD]  dv_new
  bf16* dws = dus + 64 * LD;          // [64][LD]  dw
  bf16* bks = dws + 64 * LD;          // beta k e^G
  bf16* bvs = bks + 64 * LD;          // beta v
  float* bs = (float*)(bvs + 64 * LD);    // [64]
  float* dbs = bs + 64;               // [64]
  const int chunk = blockIdx.x, h = blockIdx.y;
  const int t0 = chunk_start[chunk], len = chunk_len[chunk];
  if (len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const long long cbase = ((long long)chunk * H + h) * 64;

  if (tid < 64) { bs[tid] = tid < len ? beta[(long long)(t0 + tid) * H + h] : 0.f; dbs[tid] = 0.f; }
  for (int idx = tid; idx < 64 * 8; idx += 256) {
    const int r = idx >> 3, c8 = (idx & 7) * 8;
    cp_async16(Xb + r * LX + c8, Ainv + (cbase + r) * 64 + c8);
  }
  for (int idx = tid; idx < 64 * (DK / 8); idx += 256) {
    const int r = idx >> 4, c8 = (idx & 15) * 8;
    cp_async16(dus + r * LD + c8, dvn + (cbase + r) * DK + c8);
    cp_async16(dws + r * LD + c8, dw + (cbase + r) * DK + c8);
  }
  cp_async_commit();
  __syncthreads();                                 // bs visible
  for (int idx = tid; idx < 64 * (DK / 8); idx += 256) {
    const int i = idx >> 4, c8 = (idx & 15) * 8;
    uint4 kq = make_uint4(0, 0, 0, 0), vq = kq;
    if (i < len) {
      const long long off = ((long long)(t0 + i) * H + h) * DK + c8;
      kq = *(const uint4*)(k + off); vq = *(const uint4*)(v + off);
    }
    const float4 g0 = *(const float4*)(G + (cbase + i) * DK + c8), g1 = *(const float4*)(G + (cbase + i) * DK + c8 + 4);
    const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const __nv_bfloat162* kb = (const __nv_bfloat162*)&kq; const __nv_bfloat162* vb = (const __nv_bfloat162*)&vq;
    uint4 ok, ov;
    unsigned* okw = (unsigned*)&ok; unsigned* ovw = (unsigned*)&ov;
    const float b = bs[i];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 kf = __bfloat1622float2(kb[e]), vf = __bfloat1622float2(vb[e]);
      okw[e] = kda_pack2(b * kf.x * __expf(gv[2 * e]), b * kf.y * __expf(gv[2 * e + 1]));
      ovw[e] = kda_pack2(b * vf.x, b * vf.y);
    }
    *(uint4*)(bks + i * LD + c8) = ok;
    *(uint4*)(bvs + i * LD + c8) = ov;
  }
  cp_async_wait_all();
  __syncthreads();
  // ---- dX = du bv^T + dw bk^T  (only the lower triangle feeds dAkk); 16x16 tiles (rt, ct)
  for (int t = warp; t < 16; t += 8) {
    const int rt = t >> 2, ct = t & 3;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    if (ct <= rt) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        unsigned a[4], b[4];
        kda_frag_a(a, dus, LD, rt * 16, kk * 16, lane);
        kda_frag_bt2(b, bvs, LD, ct * 16, kk * 16, lane);
        kda_mma16816(acc[0], a, b[0], b[1]); kda_mma16816(acc[1], a, b[2], b[3]);
        kda_frag_a(a, dws, LD, rt * 16, kk * 16, lane);
        kda_frag_bt2(b, bks, LD, ct * 16, kk * 16, lane);
        kda_mma16816(acc[0], a, b[0], b[1]); kda_mma16816(acc[1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        *(unsigned*)(dXb + (rt * 16 + g + hh * 8) * LX + ct * 16 + n * 8 + 2 * t4) = kda_pack2(acc[n][2 * hh], acc[n][2 * hh + 1]);
  }
  __syncthreads();
  // ---- Y = X^T dX
  for (int t = warp; t < 16; t += 8) {
    const int rt = t >> 2, ct = t & 3;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int kt = rt; kt < 4; ++kt) {              // X^T[i,m] = X[m,i], non-zero for m >= i
      unsigned a[4], b[4];
      kda_frag_a_t(a, Xb, LX, rt * 16, kt * 16, lane);
      kda_frag_b2(b, dXb, LX, kt * 16, ct * 16, lane);
      kda_mma16816(acc[0], a, b[0], b[1]); kda_mma16816(acc[1], a, b[2], b[3]);
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        *(unsigned*)(Yb + (rt * 16 + g + hh * 8) * LX + ct * 16 + n * 8 + 2 * t4) = kda_pack2(acc[n][2 * hh], acc[n][2 * hh + 1]);
  }
  __syncthreads();
  // ---- dM = -Y X^T ; dAkk = strict_lower(dM) ; dKK = beta_i dAkk ; dbeta_i += sum_j dAkk Akk / beta_i
  for (int t = warp; t < 16; t += 8) {
    const int rt = t >> 2, ct = t & 3;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    if (ct <= rt) {
      for (int kt = 0; kt <= ct; ++kt) {           // X^T[n,j] = X[j,n], non-zero for n <= j
        unsigned a[4], b[4];
        kda_frag_a(a, Yb, LX, rt * 16, kt * 16, lane);
        kda_frag_bt2(b, Xb, LX, ct * 16, kt * 16, lane);
        kda_mma16816(acc[0], a, b[0], b[1]); kda_mma16816(acc[1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int i = rt * 16 + g + hh * 8;
      const float bi = bs[i];
      float rowsum = 0.f;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        const int j = ct * 16 + n * 8 + 2 * t4;
        const float d0 = j < i ? -acc[n][2 * hh] : 0.f, d1 = j + 1 < i ? -acc[n][2 * hh + 1] : 0.f;
        const float2 av = __bfloat1622float2(*(const __nv_bfloat162*)(Akk + (cbase + i) * 64 + j));
        rowsum += d0 * av.x + d1 * av.y;
        *(unsigned*)(dKK_out + (cbase + i) * 64 + j) = kda_pack2(d0 * bi, d1 * bi);
      }
      rowsum += __shfl_xor_sync(0xFFFFFFFFu, rowsum, 1);
      rowsum += __shfl_xor_sync(0xFFFFFFFFu, rowsum, 2);
      if (t4 == 0 && bi > 0.f) atomicAdd(&dbs[i], rowsum / bi);
    }
  }
  // ---- dbv = X^T du -> dv, dbeta ;  dbk = X^T dw -> consumed by the A-matrix kernel
  {
    const int which = warp >> 2, rt = warp & 3;
    const bf16* B = which ? dws : dus;
    float acc[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) { acc[n][0] = 0.f; acc[n][1] = 0.f; acc[n][2] = 0.f; acc[n][3] = 0.f; }
    for (int kt = rt; kt < 4; ++kt) {
      unsigned a[4];
      kda_frag_a_t(a, Xb, LX, rt * 16, kt * 16, lane);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        unsigned b[4];
        kda_frag_b2(b, B, LD, kt * 16, np * 16, lane);
        kda_mma16816(acc[2 * np], a, b[0], b[1]); kda_mma16816(acc[2 * np + 1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int i = rt * 16 + g + hh * 8;
      if (!which) {
        // dv = beta * dbv ; dbeta += sum_c v * dbv  (v recovered from the beta*v tile)
        const float bi = bs[i], inv_b = bi > 0.f ? 1.f / bi : 0.f;
        float rowsum = 0.f;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          const int c = n * 8 + 2 * t4;
          const float v0 = acc[n][2 * hh], v1 = acc[n][2 * hh + 1];
          const float2 bv = __bfloat1622float2(*(const __nv_bfloat162*)(bvs + i * LD + c));
          rowsum += (bv.x * v0 + bv.y * v1) * inv_b;
          if (i < len) *(unsigned*)(dv_out + ((long long)(t0 + i) * H + h) * DK + c) = kda_pack2(bi * v0, bi * v1);
        }
        rowsum += __shfl_xor_sync(0xFFFFFFFFu, rowsum, 1);
        rowsum += __shfl_xor_sync(0xFFFFFFFFu, rowsum, 2);
        if (t4 == 0 && i < len) atomicAdd(&dbs[i], rowsum);
      } else {
#pragma unroll
        for (int n = 0; n < 16; ++n)
          *(unsigned*)(dbk_out + (cbase + i) * DK + n * 8 + 2 * t4) = kda_pack2(acc[n][2 * hh], acc[n][2 * hh + 1]);
      }
    }
  }
  __syncthreads();
  if (tid < len) dbeta_out[(long long)(t0 + tid) * H + h] = dbs[tid];
}
constexpr int kda_bwd_wy_mma_smem() { return 3 * 64 * 72 * 2 + 4 * 64 * 136 * 2 + 128 * 4 + 128; }

// =================================================================================================== A matrices
template <int DK>
__global__ void __launch_bounds__(4 * DK, 1)
kda_bwd_amat_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const float* __restrict__ G,
                    const float* __restrict__ beta, const bf16* __restrict__ dbk,
                    const bf16* __restrict__ dKK, const bf16* __restrict__ dAqk, const float* __restrict__ dq_acc,
                    const float* __restrict__ dk_acc, const float* __restrict__ dG_acc,
                    const int* __restrict__ chunk_start, const int* __restrict__ chunk_len, int H,
                    bf16* __restrict__ dq_out, bf16* __restrict__ dk_out, float* __restrict__ dg_out,
                    float* __restrict__ dbeta_out) {
  constexpr int LD = DK + 8, NT = DK / 16, LQ = DK + 4;
  constexpr int NTHR = 4 * DK, NWARP = NTHR / 32;
  constexpr int RPT = 16;                     // rows owned by a thread: one diagonal block
  constexpr int NB = 1;
  extern __shared__ __align__(128) uint8_t smem[];
  float* Gs = (float*)smem;                   // [64][DK]
  float* stQ = Gs + 64 * DK;                  // [48][LQ]
  float* stK = stQ + 48 * LQ;                 // [48][LQ]
  float* stC = stK + 48 * LQ;                 // [16][LQ]
  float* carry = stC + 16 * LQ;               // [4][DK]
  bf16* qs = (bf16*)(carry + 4 * DK);         // [64][LD]
  bf16* ks = qs + 64 * LD;
  bf16* T1 = ks + 64 * LD;                    // Rq
  bf16* T2 = T1 + 64 * LD;                    // Rk
  bf16* Ck = T2 + 64 * LD;                    // [16][LD]
  bf16* D1 = Ck + 16 * LD;                    // [64][72]  dKK
  bf16* D2 = D1 + 64 * 72;                    // [64][72]  dAqk
  float* bs = (float*)(D2 + 64 * 72);         // [64] beta
  float* dbs = bs + 64;                       // [64] k part of dbeta
  const int chunk = blockIdx.x, h = blockIdx.y;
  const int t0 = chunk_start[chunk], len = chunk_len[chunk];
  if (len == 0) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const long long cbase = ((long long)chunk * H + h) * 64;
  const int c = tid % DK, rh = tid / DK, row0 = rh * RPT;

  for (int idx = tid; idx < 64 * (DK / 8); idx += NTHR) {
    int r = idx / (DK / 8), c8 = (idx % (DK / 8)) * 8;
    uint4 zq = make_uint4(0, 0, 0, 0), zk = zq;
    if (r < len) {
      long long off = ((long long)(t0 + r) * H + h) * DK + c8;
      zq = *(const uint4*)(q + off); zk = *(const uint4*)(k + off);
    }
    *(uint4*)(qs + r * LD + c8) = zq; *(uint4*)(ks + r * LD + c8) = zk;
  }
  for (int idx = tid; idx < 64 * (DK / 4); idx += NTHR) {
    int r = idx / (DK / 4), c4 = (idx % (DK / 4)) * 4;
    *(float4*)(Gs + r * DK + c4) = *(const float4*)(G + (cbase + r) * DK + c4);
  }
  for (int idx = tid; idx < 64 * 8; idx += NTHR) {
    int r = idx >> 3, c8 = (idx & 7) * 8;
    *(uint4*)(D1 + r * 72 + c8) = *(const uint4*)(dKK + (cbase + r) * 64 + c8);
    *(uint4*)(D2 + r * 72 + c8) = *(const uint4*)(dAqk + (cbase + r) * 64 + c8);
  }
  if (tid < 64) { bs[tid] = tid < len ? beta[(long long)(t0 + tid) * H + h] : 0.f; dbs[tid] = 0.f; }
  float dq[RPT], dk[RPT], dG[RPT];
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    long long off = (cbase + row0 + ii) * DK + c;
    dq[ii] = dq_acc[off]; dk[ii] = dk_acc[off]; dG[ii] = dG_acc[off];
  }
  __syncthreads();
  // exact diagonal blocks: this thread owns channel c of rows row0 .. row0+RPT-1
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    float Gv[16], kv[16], qv[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      int i = row0 + b * 16 + r;
      Gv[r] = Gs[i * DK + c]; kv[r] = __bfloat162float(ks[i * LD + c]); qv[r] = __bfloat162float(qs[i * LD + c]);
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) {
#pragma unroll
      for (int s = 0; s < 16; ++s) {
        if (s <= r) {
          const int i = row0 + b * 16 + r, j = row0 + b * 16 + s;
          const float d1 = s < r ? __bfloat162float(D1[i * 72 + j]) : 0.f;
          const float d2 = __bfloat162float(D2[i * 72 + j]);
          const float e = __expf(Gv[r] - Gv[s]);
          const float tk = d1 * kv[s] * e, tq = d2 * kv[s] * e;      // -> dk_i, dq_i
          const float tj = (d1 * kv[r] + d2 * qv[r]) * e;            // -> dk_j
          dk[b * 16 + r] += tk; dq[b * 16 + r] += tq; dk[b * 16 + s] += tj;
          const float gg = tk * kv[r] + tq * qv[r];
          dG[b * 16 + r] += gg; dG[b * 16 + s] -= gg;
        }
      }
    }
  }
  // off-diagonal blocks, column block J anchored at its last row (same factorisation as the forward)
  for (int J = 0; J < 3; ++J) {
    const int e = 16 * J + 15, r0 = 16 * (J + 1), nrows = 64 - r0;
    __syncthreads();
    for (int idx = tid; idx < 16 * DK; idx += NTHR) {
      int jj = idx / DK, cc = idx % DK, j = 16 * J + jj;
      Ck[jj * LD + cc] = __float2bfloat16(__bfloat162float(ks[j * LD + cc]) * __expf(Gs[e * DK + cc] - Gs[j * DK + cc]));
    }
    for (int idx = tid; idx < nrows * DK; idx += NTHR) {
      int rr = idx / DK, cc = idx % DK, i = r0 + rr;
      float f = __expf(Gs[i * DK + cc] - Gs[e * DK + cc]);
      T1[rr * LD + cc] = __float2bfloat16(__bfloat162float(qs[i * LD + cc]) * f);
      T2[rr * LD + cc] = __float2bfloat16(__bfloat162float(ks[i * LD + cc]) * f);
    }
    __syncthreads();
    const int nrt = nrows / 16;
    // dRq = D2[rows, J] Ck ; dRk = D1[rows, J] Ck ; dCk = D1[rows, J]^T Rk + D2[rows, J]^T Rq
    for (int t = warp; t < (2 * nrt + 1) * NT; t += NWARP) {
      const int kind = t / NT, nt = t % NT;
      FragC acc; wmma::fill_fragment(acc, 0.f);
      if (kind < 2 * nrt) {
        const int rt = kind >> 1, which = kind & 1;
        FragA a; FragB b;
        wmma::load_matrix_sync(a, (which ? D1 : D2) + (r0 + rt * 16) * 72 + 16 * J, 72);
        wmma::load_matrix_sync(b, Ck + nt * 16, LD);
        wmma::mma_sync(acc, a, b, acc);
        wmma::store_matrix_sync((which ? stK : stQ) + rt * 16 * LQ + nt * 16, acc, LQ, wmma::mem_row_major);
      } else {
        for (int kt = 0; kt < nrt; ++kt) {
          FragAT a; FragB b;
          wmma::load_matrix_sync(a, D1 + (r0 + kt * 16) * 72 + 16 * J, 72);
          wmma::load_matrix_sync(b, T2 + kt * 16 * LD + nt * 16, LD);
          wmma::mma_sync(acc, a, b, acc);
          wmma::load_matrix_sync(a, D2 + (r0 + kt * 16) * 72 + 16 * J, 72);
          wmma::load_matrix_sync(b, T1 + kt * 16 * LD + nt * 16, LD);
          wmma::mma_sync(acc, a, b, acc);
        }
        wmma::store_matrix_sync(stC + nt * 16, acc, LQ, wmma::mem_row_major);
      }
    }
    __syncthreads();
    const float Ge = Gs[e * DK + c];
#pragma unroll
    for (int ii = 0; ii < RPT; ++ii) {
      const int i = row0 + ii;
      if (i >= r0) {
        const float f = __expf(Gs[i * DK + c] - Ge);
        const float dRq = stQ[(i - r0) * LQ + c], dRk = stK[(i - r0) * LQ + c];
        const float qi = __bfloat162float(qs[i * LD + c]) * f, ki = __bfloat162float(ks[i * LD + c]) * f;
        dq[ii] += dRq * f; dk[ii] += dRk * f;
        dG[ii] += dRq * qi + dRk * ki;
      } else if (i >= 16 * J) {
        const float fc = __expf(Ge - Gs[i * DK + c]);
        const float dC = stC[(i - 16 * J) * LQ + c];
        dk[ii] += dC * fc;
        dG[ii] -= dC * __bfloat162float(ks[i * LD + c]) * fc;
      }
    }
  }
  // backward of w = Ainv (beta k e^G): dbk = Ainv^T dw arrives from the WY kernel
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = row0 + ii;
    const float eG = __expf(Gs[i * DK + c]);
    const float d = __bfloat162float(dbk[(cbase + i) * DK + c]);
    const float ke = __bfloat162float(ks[i * LD + c]) * eG;
    dk[ii] += bs[i] * eG * d;
    dG[ii] += bs[i] * ke * d;
    float part = ke * d;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
    if ((tid & 31) == 0) atomicAdd(&dbs[i], part);
  }
  // dg = reverse cumsum of dG over the chunk rows
  float tot = 0.f;
#pragma unroll
  for (int ii = RPT - 1; ii >= 0; --ii) { tot += dG[ii]; dG[ii] = tot; }
  carry[rh * DK + c] = tot;
  __syncthreads();
  float add = 0.f;
  for (int r2 = rh + 1; r2 < NTHR / DK; ++r2) add += carry[r2 * DK + c];
#pragma unroll
  for (int ii = 0; ii < RPT; ++ii) {
    const int i = row0 + ii;
    if (i < len) {
      long long toff = ((long long)(t0 + i) * H + h) * DK + c;
      dq_out[toff] = __float2bfloat16(dq[ii]); dk_out[toff] = __float2bfloat16(dk[ii]); dg_out[toff] = dG[ii] + add;
    }
  }
  __syncthreads();
  if (tid < len) dbeta_out[(long long)(t0 + tid) * H + h] += dbs[tid];
}
template <int DK>
constexpr int kda_bwd_amat_smem() {
  return 64 * DK * 4 + (48 + 48 + 16) * (DK + 4) * 4 + 4 * DK * 4 + 4 * 64 * (DK + 8) * 2 + 16 * (DK + 8) * 2 +
         2 * 64 * 72 * 2 + 128 * 4 + 128;
}

}  // namespace hippo

using namespace hippo;

// HIPPO_KDA_STATE_MMA=0 selects the WMMA state kernel for head_dim 128 as well (it always serves head_dim 64)
static bool kda_bwd_state_mma_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("HIPPO_KDA_STATE_MMA"); v = (e && e[0] == '0') ? 0 : 1; }
  return v == 1;
}

template <int DK>
static int launch_bwd(const void* q, const void* k, const void* v, const float* beta, const float* G, const void* w,
                      const void* qg, const void* kg, const void* Aqk, const void* Ainv, const void* Akk,
                      const void* vnew, const void* Sst, const void* d_o, const float* dfinal, const int* cs,
                      const int* cl, const int* sc, const int* so, int NC, int N, int H, void* dvn, void* dSst, void* dw, void* dAqk,
                      void* dKK, void* dbk, float* dq_acc, float* dk_acc, float* dG_acc, void* dq, void* dk, void* dv,
                      float* dg, float* dbeta, float* dh0, cudaStream_t s) {
  constexpr int VS = 32;
  auto k3 = kda_bwd_state_kernel<DK, VS>;
  auto k4a = kda_bwd_dqkw_kernel<DK>;
  auto k4b = kda_bwd_wy_kernel<DK>;
  auto k4c = kda_bwd_amat_kernel<DK>;
  static bool once = false;
  if (!once) {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_bwd_state_smem<DK, VS>())) != cudaSuccess) return (int)e;
    if ((e = cudaFuncSetAttribute(k4a, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_bwd_dqkw_smem<DK>())) != cudaSuccess) return (int)e;
    if ((e = cudaFuncSetAttribute(k4b, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_bwd_wy_smem<DK>())) != cudaSuccess) return (int)e;
    if ((e = cudaFuncSetAttribute(k4c, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_bwd_amat_smem<DK>())) != cudaSuccess) return (int)e;
    once = true;
  }
  if (NC == 0) return 0;
  if (DK == 128 && kda_bwd_state_mma_enabled()) {
    auto k3m = kda_bwd_state_mma_kernel<VS>;
    static bool once3 = false;
    if (!once3) {
      cudaError_t e = cudaFuncSetAttribute(k3m, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_bwd_state_mma_smem<VS>());
      if (e != cudaSuccess) return (int)e;
      once3 = true;
    }
    k3m<<<dim3(DK / VS, H, N), 256, kda_bwd_state_mma_smem<VS>(), s>>>((const bf16*)w, (const bf16*)qg, (const bf16*)kg,
        (const bf16*)Aqk, G, (const bf16*)d_o, cs, cl, sc, so, H, dfinal, (bf16*)dvn, (bf16*)dSst, dh0);
  } else
  k3<<<dim3(DK / VS, H, N), 256, kda_bwd_state_smem<DK, VS>(), s>>>((const bf16*)w, (const bf16*)qg, (const bf16*)kg,
      (const bf16*)Aqk, G, (const bf16*)d_o, cs, cl, sc, so, H, dfinal, (bf16*)dvn, (bf16*)dSst, dh0);
  if (DK == 128 && kda_bwd_state_mma_enabled()) {
    static bool once4 = false;
    if (!once4) {
      cudaError_t e = cudaFuncSetAttribute(kda_bwd_dqkw_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_bwd_dqkw_mma_smem());
      if (e != cudaSuccess) return (int)e;
      once4 = true;
    }
    kda_bwd_dqkw_mma_kernel<<<dim3(NC, H), 512, kda_bwd_dqkw_mma_smem(), s>>>((const bf16*)d_o, (const bf16*)vnew,
        (const bf16*)dvn, (const bf16*)Sst, (const bf16*)dSst, (const bf16*)qg, (const bf16*)kg, G, cs, cl, H, dq_acc, dk_acc,
        dG_acc, (bf16*)dw, (bf16*)dAqk);
  } else
  k4a<<<dim3(NC, H), 512, kda_bwd_dqkw_smem<DK>(), s>>>((const bf16*)d_o, (const bf16*)vnew, (const bf16*)dvn,
      (const bf16*)Sst, (const bf16*)dSst, (const bf16*)qg, (const bf16*)kg, G, cs, cl, H, dq_acc, dk_acc, dG_acc,
      (bf16*)dw, (bf16*)dAqk);
  if (DK == 128 && kda_bwd_state_mma_enabled()) {
    static bool once5 = false;
    if (!once5) {
      cudaError_t e = cudaFuncSetAttribute(kda_bwd_wy_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kda_bwd_wy_mma_smem());
      if (e != cudaSuccess) return (int)e;
      once5 = true;
    }
    kda_bwd_wy_mma_kernel<<<dim3(NC, H), 256, kda_bwd_wy_mma_smem(), s>>>((const bf16*)k, (const bf16*)v, beta, G,
        (const bf16*)Ainv, (const bf16*)Akk, (const bf16*)dvn, (const bf16*)dw, cs, cl, H, (bf16*)dbk, (bf16*)dv, dbeta, (bf16*)dKK);
  } else
  k4b<<<dim3(NC, H), 256, kda_bwd_wy_smem<DK>(), s>>>((const bf16*)k, (const bf16*)v, beta, G, (const bf16*)Ainv,
      (const bf16*)Akk, (const bf16*)dvn, (const bf16*)dw, cs, cl, H, (bf16*)dbk, (bf16*)dv, dbeta, (bf16*)dKK);
  k4c<<<dim3(NC, H), 4 * DK, kda_bwd_amat_smem<DK>(), s>>>((const bf16*)q, (const bf16*)k, G, beta, (const bf16*)dbk,
      (const bf16*)dKK, (const bf16*)dAqk, dq_acc, dk_acc, dG_acc, cs, cl, H, (bf16*)dq, (bf16*)dk, dg, dbeta);
  return (int)cudaGetLastError();
}

extern "C" int hippo_kda_bwd(const void* q, const void* k, const void* v, const float* beta, const float* G,
                             const void* w, const void* qg, const void* kg, const void* Aqk, const void* Ainv,
                             const void* Akk, const void* vnew, const void* Sst, const void* d_o, const float* dfinal,
                             const int* chunk_start, const int* chunk_len, const int* seq_chunk, const int* seq_order,
                             int NC, int N, int H, int DK, void* dvn, void* dSst, void* dw, void* dAqk, void* dKK, void* dbk, float* dq_acc,
                             float* dk_acc, float* dG_acc, void* dq, void* dk, void* dv, float* dg, float* dbeta,
                             float* dh0, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (DK == 128) return launch_bwd<128>(q, k, v, beta, G, w, qg, kg, Aqk, Ainv, Akk, vnew, Sst, d_o, dfinal, chunk_start, chunk_len, seq_chunk, seq_order, NC, N, H, dvn, dSst, dw, dAqk, dKK, dbk, dq_acc, dk_acc, dG_acc, dq, dk, dv, dg, dbeta, dh0, s);
  if (DK == 64) return launch_bwd<64>(q, k, v, beta, G, w, qg, kg, Aqk, Ainv, Akk, vnew, Sst, d_o, dfinal, chunk_start, chunk_len, seq_chunk, seq_order, NC, N, H, dvn, dSst, dw, dAqk, dKK, dbk, dq_acc, dk_acc, dG_acc, dq, dk, dv, dg, dbeta, dh0, s);
  return -1;
}
