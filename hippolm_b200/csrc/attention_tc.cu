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
// head_dim 64. Every wait is bounded. The reference has no softmax-attention layer.
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

// =====================================================================================================================
// Backward. delta = rowsum(dO * O) first, then two kernels with no atomics:
//   dQ kernel   one CTA per (query tile i, head): for every key tile j <= i   S = Q K^T, dP = dO V^T (TMEM),
//               thread = query row: P = exp2(scale S - lse), dS = scale P (dP - delta) -> bf16 K-major tile in shared
//               memory, dQ += dS K_j accumulated in TMEM over j.
//   dKV kernel  one CTA per (key tile j, head): for every query tile i >= j of the document the TRANSPOSED products
//               S^T = K Q^T and dP^T = V dO^T (TMEM lanes = keys), thread = key row writes P^T and dS^T rows, then
//               dV += P^T dO_i and dK += dS^T Q_i accumulate in TMEM over i.
// A 128 x 128 tile loaded by TMA as two 64-column swizzle atoms serves both operand roles: K-major (rows = M/N,
// descriptor step 32 B per 16 columns, atoms 16 KB apart) and MN-major (columns = M/N, rows = contraction,
// descriptor step 2048 B per 16 rows, 64-column groups 16 KB apart), so Q, dO and K are staged once per use.
struct BwdParams {
  const int* tile_start; const int* tile_len; const int* tile_seq0; const int* tile_seq_end;
  int H; long long T; float scale_log2, scale;
  const float* lse; const float* delta;
  __nv_bfloat16* dq; __nv_bfloat16* dk; __nv_bfloat16* dv;
};

__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, long long rows) {
  long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint2 a = *(const uint2*)(o + row * DH + lane * 4), b = *(const uint2*)(d_o + row * DH + lane * 4);
  const __nv_bfloat162* ab = (const __nv_bfloat162*)&a; const __nv_bfloat162* bb = (const __nv_bfloat162*)&b;
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < 2; ++e) { float2 x = __bfloat1622float2(ab[e]), y = __bfloat1622float2(bb[e]); s += x.x * y.x + x.y * y.y; }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
  if (lane == 0) delta[row] = s;
}

// one thread's 32 consecutive bf16 pairs of a K-major 128-column tile row: columns [c, c+32) of row r
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int r, int c, const uint32_t (&pk)[16]) {
  uint8_t* prow = tile + (c >> 6) * 16384 + r * 128;
#pragma unroll
  for (int q4 = 0; q4 < 4; ++q4) {
    const int piece = ((c & 63) >> 3) + q4;
    *(uint4*)(prow + ((piece ^ (r & 7)) << 4)) = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
  }
}
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int kk) {       // 16 contraction columns per step
  return make_smem_desc(base + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int kk) {      // 16 contraction rows per step
  return make_smem_desc(base + kk * 2048, 16384, 1024);
}
__device__ __forceinline__ void load_tile_128(uint8_t* dst, const CUtensorMap* map, uint64_t* bar, int x0, int row0) {
  tma_load_2d(dst, map, bar, x0, row0);
  tma_load_2d(dst + 16384, map, bar, x0 + 64, row0);
}

// ------------------------------------------------------------------------------------------------------------ dQ
// smem: Q | dO | K[2] | V[2] | dS   (7 tiles)
constexpr int SMEM_DQ = 7 * TILE_BYTES + 1024 + 256;

__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                      const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem; uint8_t* sDO = smem + TILE_BYTES;
  uint8_t* sK = smem + 2 * TILE_BYTES; uint8_t* sV = smem + 4 * TILE_BYTES; uint8_t* sDS = smem + 6 * TILE_BYTES;
  uint64_t* bars = (uint64_t*)(smem + 7 * TILE_BYTES);
  uint64_t* q_full = bars;           // 1
  uint64_t* kv_full = bars + 1;      // 2
  uint64_t* kv_empty = bars + 3;     // 2
  uint64_t* sd_full = bars + 5;      // S and dP ready in TMEM
  uint64_t* sd_empty = bars + 6;     // (4 arrivals) softmax warps have read them
  uint64_t* ds_full = bars + 7;      // (4 arrivals) dS tile written
  uint64_t* ds_empty = bars + 8;     // dQ MMA has consumed the dS tile
  uint64_t* dq_full = bars + 9;
  uint32_t* tmem_slot = (uint32_t*)(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;
  const int t0 = p.tile_start[tile], len = p.tile_len[tile], seq0 = p.tile_seq0[tile];
  if (len == 0) return;
  const int nkv = (t0 - seq0) / BKV + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    mbar_init(sd_full, 1); mbar_init(sd_empty, 4); mbar_init(ds_full, 4); mbar_init(ds_empty, 1); mbar_init(dq_full, 1);
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dQ = tmem_base + 256;
  const int x0 = h * DH;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
      load_tile_128(sQ, &tmQ, q_full, x0, t0);
      load_tile_128(sDO, &tmDO, q_full, x0, t0);
      bool ok = true;
      for (int j = 0; j < nkv && ok; ++j) {
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        ok = mbar_wait(&kv_empty[st], ph ^ 1, kWaitSmemEmpty, j);
        if (!ok) break;
        mbar_expect_tx(&kv_full[st], 2 * TILE_BYTES);
        load_tile_128(sK + st * TILE_BYTES, &tmK, &kv_full[st], x0, seq0 + j * BKV);
        load_tile_128(sV + st * TILE_BYTES, &tmV, &kv_full[st], x0, seq0 + j * BKV);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_nt = make_idesc_f16(128, 128, 1, 0, 0);
      constexpr uint32_t idesc_nn = make_idesc_f16(128, 128, 1, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aDO = smem_u32(sDO), aDS = smem_u32(sDS);
      bool ok = mbar_wait(q_full, 0, kWaitTmaFull, 9000);
      for (int j = 0; j < nkv && ok; ++j) {
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        ok = mbar_wait(&kv_full[st], ph, kWaitTmaFull, j);
        if (ok) ok = mbar_wait(sd_empty, (j & 1) ^ 1, kWaitTmemEmpty, j);
        if (!ok) break;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * TILE_BYTES), aV = smem_u32(sV + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_f16_ss(tmem_S, desc_kmajor(aQ, kk), desc_kmajor(aK, kk), idesc_nt, kk ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_f16_ss(tmem_dP, desc_kmajor(aDO, kk), desc_kmajor(aV, kk), idesc_nt, kk ? 1u : 0u);
        tc_commit(sd_full);
        ok = mbar_wait(ds_full, j & 1, kWaitGeneric, j);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)      // dQ += dS (K-major, keys contracted) x K_j (MN-major: head dim = N)
          mma_f16_ss(tmem_dQ, desc_kmajor(aDS, kk), desc_mnmajor(aK, kk), idesc_nn, (j | kk) ? 1u : 0u);
        tc_commit(&kv_empty[st]);
        tc_commit(ds_empty);
      }
      if (ok) tc_commit(dq_full);
    }
  } else {
    const int qd = warp & 3, r = qd * 32 + lane;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const long long tok = (long long)t0 + r;
    const bool in_range = tok < p.T;
    const float lse_r = in_range ? p.lse[tok * p.H + h] : 0.f;
    const float delta_r = in_range ? p.delta[tok * p.H + h] : 0.f;
    bool ok = true;
    for (int j = 0; j < nkv && ok; ++j) {
      ok = mbar_wait(sd_full, j & 1, kWaitTmemFull, j);
      if (ok) ok = mbar_wait(ds_empty, (j & 1) ^ 1, kWaitSmemEmpty, 4000 + j);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool diag = (j == nkv - 1);
#pragma unroll 1
      for (int c = 0; c < BKV; c += 32) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem_S + lane_off + c, sv);
        tmem_ld_32x32(tmem_dP + lane_off + c, dv);
        tc_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float d2[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const float pr = (diag && c + e + u > r) ? 0.f : exp2f(__uint_as_float(sv[e + u]) * p.scale_log2 - lse_r);
            d2[u] = pr * (__uint_as_float(dv[e + u]) - delta_r) * p.scale;
          }
          __nv_bfloat162 b2 = __floats2bfloat162_rn(d2[0], d2[1]);
          pk[e >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
        store_row_chunk(sDS, r, c, pk);
      }
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) { mbar_arrive(sd_empty); mbar_arrive(ds_full); }
    }
    if (ok) ok = mbar_wait(dq_full, 0, kWaitTmemFull, 7000);
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (ok) {
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < DH; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_dQ + lane_off + c, v);
        tc_wait_ld();
        if (r < len) {
          uint4* dst = (uint4*)(p.dq + (tok * p.H + h) * DH + c);
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            __nv_bfloat162* wb = (__nv_bfloat162*)&w;
#pragma unroll
            for (int e = 0; e < 4; ++e)
              wb[e] = __floats2bfloat162_rn(__uint_as_float(v[8 * q4 + 2 * e]), __uint_as_float(v[8 * q4 + 2 * e + 1]));
            dst[q4] = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ------------------------------------------------------------------------------------------------------------ dK, dV
// smem: K | V | Q | dO | P^T | dS^T   (6 tiles) + lse / delta of the current query tile
constexpr int SMEM_DKV = 6 * TILE_BYTES + 1024 + 1024 + 256;

__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                       const __grid_constant__ BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem; uint8_t* sV = smem + TILE_BYTES; uint8_t* sQ = smem + 2 * TILE_BYTES; uint8_t* sDO = smem + 3 * TILE_BYTES;
  uint8_t* sPT = smem + 4 * TILE_BYTES; uint8_t* sDST = smem + 5 * TILE_BYTES;
  float* s_lse = (float*)(smem + 6 * TILE_BYTES);           // [128]
  float* s_delta = s_lse + 128;                             // [128]
  uint64_t* bars = (uint64_t*)(smem + 6 * TILE_BYTES + 1024);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qd_full = bars + 1;      // Q_i, dO_i landed
  uint64_t* qd_empty = bars + 2;     // both accumulate MMAs of tile i have completed
  uint64_t* sd_full = bars + 3;      // S^T, dP^T ready
  uint64_t* sd_empty = bars + 4;     // (4 arrivals)
  uint64_t* pds_full = bars + 5;     // (4 arrivals) P^T and dS^T written
  uint64_t* acc_full = bars + 6;
  uint64_t* stat_full = bars + 7;    // (128 arrivals) row statistics of the query tile staged
  uint32_t* tmem_slot = (uint32_t*)(bars + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, h = blockIdx.y;                 // early key tiles (most query tiles) come first
  const int k0 = p.tile_start[tile], klen = p.tile_len[tile], seq0 = p.tile_seq0[tile], seq_end = p.tile_seq_end[tile];
  if (klen == 0) return;
  const int nq = (seq_end - k0 + BQ - 1) / BQ;                 // query tiles i >= j of this document

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(qd_full, 1); mbar_init(qd_empty, 1);
    mbar_init(sd_full, 1); mbar_init(sd_empty, 4); mbar_init(pds_full, 4); mbar_init(acc_full, 1);
    mbar_init(stat_full, 128);
    fence_barrier_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmDO);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dV = tmem_base + 256, tmem_dK = tmem_base + 384;
  const int x0 = h * DH;
  (void)seq0;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      load_tile_128(sK, &tmK, kv_full, x0, k0);
      load_tile_128(sV, &tmV, kv_full, x0, k0);
      bool ok = true;
      for (int i = 0; i < nq && ok; ++i) {
        ok = mbar_wait(qd_empty, (i & 1) ^ 1, kWaitSmemEmpty, i);
        if (!ok) break;
        mbar_expect_tx(qd_full, 2 * TILE_BYTES);
        load_tile_128(sQ, &tmQ, qd_full, x0, k0 + i * BQ);
        load_tile_128(sDO, &tmDO, qd_full, x0, k0 + i * BQ);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_nt = make_idesc_f16(128, 128, 1, 0, 0);
      constexpr uint32_t idesc_nn = make_idesc_f16(128, 128, 1, 0, 1);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aDO = smem_u32(sDO);
      const uint32_t aPT = smem_u32(sPT), aDST = smem_u32(sDST);
      bool ok = mbar_wait(kv_full, 0, kWaitTmaFull, 9000);
      for (int i = 0; i < nq && ok; ++i) {
        ok = mbar_wait(qd_full, i & 1, kWaitTmaFull, i);
        if (ok) ok = mbar_wait(sd_empty, (i & 1) ^ 1, kWaitTmemEmpty, i);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_f16_ss(tmem_S, desc_kmajor(aK, kk), desc_kmajor(aQ, kk), idesc_nt, kk ? 1u : 0u);     // S^T = K Q^T
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) mma_f16_ss(tmem_dP, desc_kmajor(aV, kk), desc_kmajor(aDO, kk), idesc_nt, kk ? 1u : 0u);   // dP^T = V dO^T
        tc_commit(sd_full);
        ok = mbar_wait(pds_full, i & 1, kWaitGeneric, i);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)      // dV += P^T (K-major, queries contracted) x dO_i (MN-major)
          mma_f16_ss(tmem_dV, desc_kmajor(aPT, kk), desc_mnmajor(aDO, kk), idesc_nn, (i | kk) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)      // dK += dS^T x Q_i (MN-major)
          mma_f16_ss(tmem_dK, desc_kmajor(aDST, kk), desc_mnmajor(aQ, kk), idesc_nn, (i | kk) ? 1u : 0u);
        tc_commit(qd_empty);                // also means: P^T / dS^T tiles are free again
      }
      if (ok) tc_commit(acc_full);
    }
  } else {
    const int qd = warp & 3, r = qd * 32 + lane;                // key row inside the tile
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    bool ok = true;
    for (int i = 0; i < nq && ok; ++i) {
      const int q0 = k0 + i * BQ;
      const int qlen = min(BQ, seq_end - q0);
      // The accumulate MMAs of tile i-1 have completed (qd_empty phase i-1): P^T / dS^T are free again, and every
      // softmax thread is past its reads of the previous tile's row statistics (it arrived on pds_full before them).
      if (i > 0) ok = mbar_wait(qd_empty, (i - 1) & 1, kWaitSmemEmpty, 4000 + i);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      {
        const long long tq = (long long)q0 + r;
        const bool in_range = r < qlen && tq < p.T;
        s_lse[r] = in_range ? p.lse[tq * p.H + h] : 0.f;
        s_delta[r] = in_range ? p.delta[tq * p.H + h] : 0.f;
      }
      mbar_arrive(stat_full);                                   // 128 arrivals: a bounded barrier of the softmax warps
      ok = mbar_wait(stat_full, i & 1, kWaitGeneric, 6000 + i);
      if (ok) ok = mbar_wait(sd_full, i & 1, kWaitTmemFull, i);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool diag = (i == 0);
#pragma unroll 1
      for (int c = 0; c < BQ; c += 32) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem_S + lane_off + c, sv);
        tmem_ld_32x32(tmem_dP + lane_off + c, dv);
        tc_wait_ld();
        uint32_t pp[16], pd[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float p2[2], d2[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int qc = c + e + u;                           // query column
            const bool masked = (diag && qc < r) || qc >= qlen;
            const float pr = masked ? 0.f : exp2f(__uint_as_float(sv[e + u]) * p.scale_log2 - s_lse[qc]);
            p2[u] = pr;
            d2[u] = pr * (__uint_as_float(dv[e + u]) - s_delta[qc]) * p.scale;
          }
          __nv_bfloat162 b2 = __floats2bfloat162_rn(p2[0], p2[1]);
          pp[e >> 1] = *reinterpret_cast<uint32_t*>(&b2);
          b2 = __floats2bfloat162_rn(d2[0], d2[1]);
          pd[e >> 1] = *reinterpret_cast<uint32_t*>(&b2);
        }
        store_row_chunk(sPT, r, c, pp);
        store_row_chunk(sDST, r, c, pd);
      }
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) { mbar_arrive(sd_empty); mbar_arrive(pds_full); }
    }
    if (ok) ok = mbar_wait(acc_full, 0, kWaitTmemFull, 7000);
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (ok) {
      tc_fence_after();
      const long long tok = (long long)k0 + r;
#pragma unroll 1
      for (int c = 0; c < 2 * DH; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem_dV + lane_off + c, v);              // dV columns [0,128), dK columns [128,256)
        tc_wait_ld();
        if (r < klen) {
          __nv_bfloat16* base = (c < DH ? p.dv : p.dk) + (tok * p.H + h) * DH + (c & (DH - 1));
          uint4* dst = (uint4*)base;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            __nv_bfloat162* wb = (__nv_bfloat162*)&w;
#pragma unroll
            for (int e = 0; e < 4; ++e)
              wb[e] = __floats2bfloat162_rn(__uint_as_float(v[8 * q4 + 2 * e]), __uint_as_float(v[8 * q4 + 2 * e + 1]));
            dst[q4] = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// tile table with `rows`-row tiles that never straddle a document
__global__ void attn_build_tiles_rows_kernel(const int* __restrict__ cu, int N, int rows, int* __restrict__ tile_start,
                                             int* __restrict__ tile_len, int* __restrict__ tile_seq0,
                                             int* __restrict__ tile_seq_end, int nt_max) {
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
      if (c < nt_max) { tile_start[c] = s; tile_len[c] = min(rows, e - s); tile_seq0[c] = s0; tile_seq_end[c] = e; }
  }
  for (int c = total + threadIdx.x; c < nt_max; c += blockDim.x) { tile_start[c] = 0; tile_len[c] = 0; tile_seq0[c] = 0; tile_seq_end[c] = 0; }
}

}  // namespace fa
}  // namespace hippo

using namespace hippo;

extern "C" int hippo_attn_build_tiles_rows(const int* cu, int N, int rows, int* ts, int* tl, int* t0, int* te, int nt_max, void* s) {
  fa::attn_build_tiles_rows_kernel<<<1, 256, (N + 1) * sizeof(int), (cudaStream_t)s>>>(cu, N, rows, ts, tl, t0, te, nt_max);
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

// Backward of hippo_attn_fwd_tc. d_o, dq, dk, dv: [T, H, 128] bf16 contiguous; delta: [T, H] fp32 scratch;
// ts / tl / t0 / te: table of 128-row tiles (start, length, document start, document end).
extern "C" int hippo_attn_bwd_tc(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                 const float* lse, float* delta, const int* ts, const int* tl, const int* t0,
                                 const int* te, int NT, int H, long long T, float scale, void* dq, void* dk, void* dv,
                                 void* stream) {
  if (NT == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  const uint64_t cols = (uint64_t)H * fa::DH;
  int rc = make_tmap_2d(&tmQ, q, cols, (uint64_t)T, cols * 2, 64, 128, 2, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmK, k, cols, (uint64_t)T, cols * 2, 64, 128, 2, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmV, v, cols, (uint64_t)T, cols * 2, 64, 128, 2, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmDO, d_o, cols, (uint64_t)T, cols * 2, 64, 128, 2, true);
  if (rc) return rc;
  const long long rows = T * H;
  fa::attn_delta_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, rows);
  fa::BwdParams p;
  p.tile_start = ts; p.tile_len = tl; p.tile_seq0 = t0; p.tile_seq_end = te; p.H = H; p.T = T;
  p.scale_log2 = scale * 1.4426950408889634f; p.scale = scale; p.lse = lse; p.delta = delta;
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(fa::attn_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa::SMEM_DQ);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(fa::attn_bwd_dkv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fa::SMEM_DKV);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  fa::attn_bwd_dq_tc_kernel<<<dim3(NT, H), fa::THREADS, fa::SMEM_DQ, st>>>(tmQ, tmK, tmV, tmDO, p);
  fa::attn_bwd_dkv_tc_kernel<<<dim3(NT, H), fa::THREADS, fa::SMEM_DKV, st>>>(tmQ, tmK, tmV, tmDO, p);
  return (int)cudaGetLastError();
}
