// Causal variable-length flash attention, forward, on tcgen05 tensor cores (sm_100a), head_dim 128.
//
// One CTA per (128-row query tile, head), 192 threads:
//   warp 0     TMA producer: Q once, then K and V tiles of 128 keys through two-stage rings
//   warp 1     MMA issuer (one thread): S = Q K^T into one of two 128-column TMEM buffers, O_j = P V into a third
//   warps 2-5  softmax: thread = query row. Reads its S row from TMEM (tcgen05.ld 32x32b), row max and sum without
//              shuffles, writes P (bf16) into shared memory in the 128-byte-swizzled K-major layout the MMA reads,
//              then folds the P V product into the fp32 output row it keeps in registers: O = alpha O + P V.
// S(j+1) is issued before P(j) V(j), so the tensor core computes the next scores while the softmax of tile j runs.
// q, k, v are packed token-major [T, H, 128] bf16 and are read through 2-D tensor maps over [T, H*128]; documents
// come from a table of 128-row tiles that never straddle a document (start, length, document start). Keys past the
// causal diagonal (which includes every key of a following document) are masked in the last tile only.
// Exp2-domain online softmax; lse = m + log2(l) as in the mma.sync kernels of attention.cu, which keep serving
// head_dim 64 and the backward pass. Every wait is bounded. The reference has no softmax-attention layer.
#include "sm100.cuh"
#include "host_utils.h"

namespace hippo {
namespace fa {

constexpr int BQ = 128, BKV = 128, DH = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;            // any 128 x 128 bf16 operand tile (two 16 KB swizzle atoms)
constexpr int THREADS = 192;
// Q | K[2] | V[2] | P | barriers
constexpr int SMEM = 6 * TILE_BYTES + 1024 + 256;

struct Params {
  const int* tile_start; const int* tile_len; const int* tile_seq0;
  int H; float scale_log2;
  __nv_bfloat16* o; float* lse;
};

__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TILE_BYTES;                   // 2 stages
  uint8_t* sV = smem + 3 * TILE_BYTES;               // 2 stages
  uint8_t* sP = smem + 5 * TILE_BYTES;
  uint64_t* bars = (uint64_t*)(smem + 6 * TILE_BYTES);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;        // 2
  uint64_t* v_empty = bars + 7;       // 2
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* s_empty = bars + 11;      // 2  (4 arrivals: one per softmax warp)
  uint64_t* p_full = bars + 13;       // 1  (4 arrivals)
  uint64_t* p_empty = bars + 14;      // 1
  uint64_t* o_full = bars + 15;       // 1
  uint64_t* o_empty = bars + 16;      // 1  (4 arrivals)
  uint32_t* tmem_slot = (uint32_t*)(bars + 17);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;       // long tiles (late in their document) first
  const int h = blockIdx.y;
  const int t0 = p.tile_start[tile], len = p.tile_len[tile], seq0 = p.tile_seq0[tile];
  if (len == 0) return;                                         // whole CTA, before any barrier or TMEM use
  const int nkv = (t0 - seq0) / BKV + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4); mbar_init(p_empty, 1); mbar_init(o_full, 1); mbar_init(o_empty, 4);
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_O = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      const int x0 = h * DH;
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_2d(sQ, &tmQ, q_full, x0, t0);
      tma_load_2d(sQ + 16384, &tmQ, q_full, x0 + 64, t0);
      bool ok = true;
      for (int j = 0; j < nkv && ok; ++j) {
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        const int kv0 = seq0 + j * BKV;
        ok = mbar_wait(&k_empty[st], ph ^ 1, kWaitSmemEmpty, j);
        if (!ok) break;
        mbar_expect_tx(&k_full[st], TILE_BYTES);
        tma_load_2d(sK + st * TILE_BYTES, &tmK, &k_full[st], x0, kv0);
        tma_load_2d(sK + st * TILE_BYTES + 16384, &tmK, &k_full[st], x0 + 64, kv0);
        ok = mbar_wait(&v_empty[st], ph ^ 1, kWaitSmemEmpty, 1000 + j);
        if (!ok) break;
        mbar_expect_tx(&v_full[st], TILE_BYTES);
        // V is the MN-major B operand of P V: per 64-key block two boxes of 64 head-dim columns x 64 keys
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
          for (int c = 0; c < 2; ++c)
            tma_load_2d(sV + st * TILE_BYTES + b * 16384 + c * 8192, &tmV, &v_full[st], x0 + c * 64, kv0 + b * 64);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(BQ, BKV, 1, 0, 0);    // Q (K-major) x K^T (K-major)
      constexpr uint32_t idesc_o = make_idesc_f16(BQ, DH, 1, 0, 1);     // P (K-major) x V (MN-major)
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, kWaitTmaFull, j)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, kWaitTmemEmpty, j)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < DH / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_f16_ss(tmem_S[st], make_smem_desc(aQ + off, 16, 1024), make_smem_desc(aK + off, 16, 1024), idesc_s, kk ? 1u : 0u);
        }
        tc_commit(&s_full[st]);
        tc_commit(&k_empty[st]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, kWaitTmaFull, 9000);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nkv && ok; ++j) {
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < nkv) { ok = issue_s(j + 1); if (!ok) break; }
        ok = mbar_wait(&v_full[st], ph, kWaitTmaFull, 2000 + j);
        if (ok) ok = mbar_wait(p_full, j & 1, kWaitGeneric, j);
        if (ok) ok = mbar_wait(o_empty, (j & 1) ^ 1, kWaitTmemEmpty, 3000 + j);
        if (!ok) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint32_t offp = (kk >> 2) * 16384 + (kk & 3) * 32;           // P: keys are the contraction, K-major
          const uint32_t offv = (kk >> 2) * 16384 + (kk & 3) * 2048;         // V: 16 key rows = 2048 bytes
          mma_f16_ss(tmem_O, make_smem_desc(aP + offp, 16, 1024), make_smem_desc(aV + offv, 8192, 1024), idesc_o, kk ? 1u : 0u);
        }
        tc_commit(o_full);
        tc_commit(&v_empty[st]);
        tc_commit(p_empty);
      }
    }
  } else {
    const int qd = warp & 3;                                  // TMEM lane quarter of this warp
    const int r = qd * 32 + lane;                             // query row inside the tile
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    float o[DH];
#pragma unroll
    for (int d = 0; d < DH; ++d) o[d] = 0.f;
    float m_i = -INFINITY, l_i = 0.f;
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
      ok = mbar_wait(&s_full[st], ph, kWaitTmemFull, j);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool diag = (j == nkv - 1);
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BKV; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_S[st] + lane_off + c, v);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float s = __uint_as_float(v[e]) * p.scale_log2;
          if (diag && c + e > r) s = -INFINITY;
          mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m_i, mx);                      // finite: column 0 of the first tile is never masked
      const float alpha = exp2f(m_i - m_new);                  // 0 on the first tile (m_i = -inf)
      m_i = m_new;
      // P(j-1) must have been consumed by its MMA before this tile's P overwrites the buffer
      ok = mbar_wait(p_empty, (j & 1) ^ 1, kWaitSmemEmpty, 4000 + j);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      // pass 2: probabilities -> bf16 -> swizzled K-major rows of the P tile
      float rs = 0.f;
#pragma unroll 1
      for (int c = 0; c < BKV; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_S[st] + lane_off + c, v);
        tc_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float s0 = __uint_as_float(v[e]) * p.scale_log2, s1 = __uint_as_float(v[e + 1]) * p.scale_log2;
          float p0 = (diag && c + e > r) ? 0.f : exp2f(s0 - m_new);
          float p1 = (diag && c + e + 1 > r) ? 0.f : exp2f(s1 - m_new);
          rs += p0 + p1;
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
          pk[e >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
        // 32 keys = four 16-byte pieces; piece index inside the 64-key atom is xor-swizzled with the row
        uint8_t* prow = sP + (c >> 6) * 16384 + r * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int piece = ((c & 63) >> 3) + q4;
          *(uint4*)(prow + ((piece ^ (r & 7)) << 4)) = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
        }
      }
      l_i = l_i * alpha + rs;
      tc_fence_before();
      fence_proxy_async();                                     // generic-proxy smem writes -> visible to the MMA
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s_empty[st]); mbar_arrive(p_full); }
      // fold P V into the running output
      ok = mbar_wait(o_full, j & 1, kWaitTmemFull, 5000 + j);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < DH; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_O + lane_off + c, v);
        tc_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c + e] = o[c + e] * alpha + __uint_as_float(v[e]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_empty);
    }
    if (ok && r < len) {
      const float inv = l_i > 0.f ? 1.f / l_i : 0.f;
      const long long tok = (long long)t0 + r;
      uint4* dst = (uint4*)(p.o + (tok * p.H + h) * DH);
#pragma unroll
      for (int d = 0; d < DH; d += 8) {
        uint4 w;
        __nv_bfloat162* wb = (__nv_bfloat162*)&w;
#pragma unroll
        for (int e = 0; e < 4; ++e) wb[e] = __floats2bfloat162_rn(o[d + 2 * e] * inv, o[d + 2 * e + 1] * inv);
        dst[d >> 3] = w;
      }
      p.lse[tok * p.H + h] = m_i + log2f(l_i);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// tile table with `rows`-row tiles that never straddle a document
__global__ void attn_build_tiles_rows_kernel(const int* __restrict__ cu, int N, int rows, int* __restrict__ tile_start,
                                             int* __restrict__ tile_len, int* __restrict__ tile_seq0, int nt_max) {
  __shared__ int total;
  extern __shared__ int first[];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int n = 0; n < N; ++n) { first[n] = acc; acc += (cu[n + 1] - cu[n] + rows - 1) / rows; }
    total = acc;
  }
  __syncthreads();
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    int s0 = cu[n], e = cu[n + 1], c = first[n];
    for (int s = s0; s < e; s += rows, ++c)
      if (c < nt_max) { tile_start[c] = s; tile_len[c] = min(rows, e - s); tile_seq0[c] = s0; }
  }
  for (int c = total + threadIdx.x; c < nt_max; c += blockDim.x) { tile_start[c] = 0; tile_len[c] = 0; tile_seq0[c] = 0; }
}

}  // namespace fa
}  // namespace hippo

using namespace hippo;

extern "C" int hippo_attn_build_tiles_rows(const int* cu, int N, int rows, int* ts, int* tl, int* t0, int nt_max, void* s) {
  fa::attn_build_tiles_rows_kernel<<<1, 256, (N + 1) * sizeof(int), (cudaStream_t)s>>>(cu, N, rows, ts, tl, t0, nt_max);
  return (int)cudaGetLastError();
}

// q, k, v, o: [T, H, 128] bf16 contiguous; ts / tl / t0: table of 128-row tiles (hippo_attn_build_tiles_rows); lse: [T, H]
extern "C" int hippo_attn_fwd_tc(const void* q, const void* k, const void* v, const int* ts, const int* tl, const int* t0,
                                 int NT, int H, long long T, float scale, void* o, float* lse, void* stream) {
  if (NT == 0) return 0;
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t cols = (uint64_t)H * fa::DH;
  int rc = make_tmap_2d(&tmQ, q, cols, (uint64_t)T, cols * 2, 64, 128, 2, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, k, cols, (uint64_t)T, cols * 2, 64, 128, 2, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v, cols, (uint64_t)T, cols * 2, 64, 64, 2, true);
  if (rc) return rc;
  fa::Params p;
  p.tile_start = ts; p.tile_len = tl; p.tile_seq0 = t0; p.H = H; p.scale_log2 = scale * 1.4426950408889634f;
  p.o = (__nv_bfloat16*)o; p.lse = lse;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fa::attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  fa::attn_fwd_tc_kernel<<<dim3(NT, H), fa::THREADS, fa::SMEM, (cudaStream_t)stream>>>(tmQ, tmK, tmV, p);
  return (int)cudaGetLastError();
}
