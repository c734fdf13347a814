// Vocab-parallel cross entropy with the cross-rank softmax reduction inside the kernels (no NCCL call).
//
// Every rank holds the logits of its vocabulary shard for a chunk of tokens, z[C, V/w] (fp32, straight from the GEMM
// epilogue). The row statistics kernel computes (max, sum exp, target logit) of its shard and stores the triple into
// EVERY rank's statistics buffer at slot [source rank][row] with plain peer stores, then releases one arrival per row
// on each destination. The gradient kernel waits (bounded) until all sources have delivered the chunk, merges the w
// triples of its row (global max, rescaled sum, target logit), adds the row's loss term and writes
// dz = (softmax - onehot) * row weight for its shard. Replaces the max / sum all-reduces of the reference's
// fused linear cross entropy (fla/modules/fused_linear_cross_entropy.py:682-708).
#include "sm100.cuh"
#include <cuda_bf16.h>

namespace hippo {

struct CeCommParams {
  int world, rank, max_rows;
  float4* stats_peer[8];            // [world][max_rows] on every rank
  uint32_t* flag_peer[8];           // [world] arrival counters on every rank, indexed by source rank
  uint32_t target;                  // counter value once every row of every call so far has arrived
  long long wait_cycles;
};

__device__ __forceinline__ float ce_wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

__global__ void __launch_bounds__(512)
ce_stats_push_kernel(const float* __restrict__ z, const long long* __restrict__ target, int V,
                     const __grid_constant__ CeCommParams cp) {
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
  s = ce_wsum(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int k = 0; k < (blockDim.x >> 5); ++k) t += sh[k];
    const long long tg = target[row];
    const float4 v = make_float4(m, t, (tg >= 0 && HIPPO_IN_BOUNDS(tg, V, 4)) ? zr[tg] : 0.f, 0.f);
    for (int d = 0; d < cp.world; ++d) {
      const int peer = (cp.rank + d) % cp.world;
      cp.stats_peer[peer][(long long)cp.rank * cp.max_rows + row] = v;
    }
    __threadfence_system();
    for (int d = 0; d < cp.world; ++d) {
      const int peer = (cp.rank + d) % cp.world;
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(cp.flag_peer[peer] + cp.rank), "r"(1u) : "memory");
    }
  }
}

__global__ void __launch_bounds__(512)
ce_grad_merge_kernel(const float* __restrict__ z, const long long* __restrict__ target, const float* __restrict__ roww,
                     __nv_bfloat16* __restrict__ dz, int V, float* __restrict__ loss_sum,
                     const __grid_constant__ CeCommParams cp) {
  __shared__ float s_lse;
  const long long row = blockIdx.x;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int src = 0; src < cp.world && ok; ++src) {
      const uint32_t* f = cp.flag_peer[cp.rank] + src;
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((int32_t)(v - cp.target) < 0) {
        // a wait that already ran out elsewhere in this launch is not repeated by the remaining row CTAs
        if (*(volatile int*)&g_status.code != 0) { ok = false; break; }
        const long long t0 = clock64();
        do {
          __nanosleep(64);
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
          if (clock64() - t0 > cp.wait_cycles) { report(kWaitPeerFlag, 200 + src); ok = false; break; }
        } while ((int32_t)(v - cp.target) < 0);
      }
    }
    float gm = -INFINITY, se = 0.f, tz = 0.f;
    const float4* st = cp.stats_peer[cp.rank];
    for (int src = 0; src < cp.world; ++src) gm = fmaxf(gm, __ldcg(&st[(long long)src * cp.max_rows + row]).x);
    for (int src = 0; src < cp.world; ++src) {
      const float4 v = __ldcg(&st[(long long)src * cp.max_rows + row]);
      se += v.y * __expf(v.x - gm);
      tz += v.z;
    }
    const float lse = gm + __logf(se);
    s_lse = ok ? lse : 0.f;
    if (ok && roww[row] > 0.f) atomicAdd(loss_sum, lse - tz);
  }
  __syncthreads();
  const float l = s_lse, w = roww[row];
  const long long tg = target[row];
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    float pr = __expf(z[row * V + c] - l);
    if (c == tg) pr -= 1.f;
    dz[row * V + c] = __float2bfloat16(pr * w);
  }
}

// ---- statistics from the logits GEMM epilogue (hippo_gemm_bf16_lce): merge of the per-tile pairs, bf16 logits
// One thread per row merges the row's (max, sum exp) pairs of all 256-column tiles (part[tile][row], so a warp reads
// consecutive addresses), stores (max, sum exp, target logit) into the statistics slot [this rank][row] of every rank and,
// once per block, releases as many arrivals as the block has rows on each destination. With world == 1 the triple only
// goes to the local buffer and no counter is touched.
__global__ void __launch_bounds__(256)
ce_part_merge_kernel(const float2* __restrict__ part, const float* __restrict__ tz, const long long* __restrict__ target,
                     long long C, int tiles_n, const __grid_constant__ CeCommParams cp) {
  const long long row = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (row < C) {
    float m = -INFINITY, s = 0.f;
    for (int t = 0; t < tiles_n; ++t) {
      const float2 v = part[(long long)t * C + row];
      if (v.x > m) { s = s * __expf(m - v.x) + v.y; m = v.x; }
      else s += v.y * __expf(v.x - m);
    }
    const float4 v = make_float4(m, s, target[row] >= 0 ? tz[row] : 0.f, 0.f);
    for (int d = 0; d < cp.world; ++d) {
      const int peer = (cp.rank + d) % cp.world;
      cp.stats_peer[peer][(long long)cp.rank * cp.max_rows + row] = v;
    }
    if (cp.world > 1) __threadfence_system();
  }
  if (cp.world == 1) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long left = C - (long long)blockIdx.x * blockDim.x;
    const uint32_t n = (uint32_t)(left < (long long)blockDim.x ? left : (long long)blockDim.x);
    for (int d = 0; d < cp.world; ++d) {
      const int peer = (cp.rank + d) % cp.world;
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(cp.flag_peer[peer] + cp.rank), "r"(n) : "memory");
    }
  }
}

// Gradient of the logits in place: z[row][c] (bf16) <- (exp(z - lse) - [c == target]) * row weight, with lse merged from
// the statistics of all ranks (bounded wait for every source when world > 1); adds lse - z_target of weighted rows to
// loss_sum. One block per row, 8 logits per thread and step.
__global__ void __launch_bounds__(256)
ce_grad_inplace_kernel(__nv_bfloat16* __restrict__ z, const long long* __restrict__ target, const float* __restrict__ roww,
                       int V, float* __restrict__ loss_sum, const __grid_constant__ CeCommParams cp) {
  __shared__ float s_lse;
  const long long row = blockIdx.x;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int src = 0; cp.world > 1 && src < cp.world && ok; ++src) {
      const uint32_t* f = cp.flag_peer[cp.rank] + src;
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((int32_t)(v - cp.target) < 0) {
        if (*(volatile int*)&g_status.code != 0) { ok = false; break; }      // a wait already ran out in this launch
        const long long t0 = clock64();
        do {
          __nanosleep(64);
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
          if (clock64() - t0 > cp.wait_cycles) { report(kWaitPeerFlag, 300 + src); ok = false; break; }
        } while ((int32_t)(v - cp.target) < 0);
      }
    }
    float gm = -INFINITY, se = 0.f, tz = 0.f;
    const float4* st = cp.stats_peer[cp.rank];
    for (int src = 0; src < cp.world; ++src) gm = fmaxf(gm, __ldcg(&st[(long long)src * cp.max_rows + row]).x);
    for (int src = 0; src < cp.world; ++src) {
      const float4 v = __ldcg(&st[(long long)src * cp.max_rows + row]);
      se += v.y * __expf(v.x - gm);
      tz += v.z;
    }
    const float lse = gm + __logf(se);
    s_lse = ok ? lse : 0.f;
    if (ok && roww[row] > 0.f) atomicAdd(loss_sum, lse - tz);
  }
  __syncthreads();
  const float l = s_lse, w = roww[row];
  const long long tg = target[row];
  uint4* zr = (uint4*)(z + row * V);                                         // V % 8 == 0: rows start 16-byte aligned
  for (int c8 = threadIdx.x; c8 < V / 8; c8 += blockDim.x) {
    uint4 v = zr[c8];
    __nv_bfloat162* vb = (__nv_bfloat162*)&v;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = __bfloat1622float2(vb[e]);
      f.x = __expf(f.x - l); f.y = __expf(f.y - l);
      const int c = c8 * 8 + 2 * e;
      if (c == tg) f.x -= 1.f;
      if (c + 1 == tg) f.y -= 1.f;
      vb[e] = __floats2bfloat162_rn(f.x * w, f.y * w);
    }
    zr[c8] = v;
  }
}

static void fill(CeCommParams& cp, void* const* stats_ptrs, void* const* flag_ptrs, int world, int rank, int max_rows,
                 unsigned target, long long wait_cycles) {
  cp.world = world; cp.rank = rank; cp.max_rows = max_rows; cp.target = target;
  cp.wait_cycles = wait_cycles > 0 ? wait_cycles : kWaitCycles;
  for (int r = 0; r < world; ++r) { cp.stats_peer[r] = (float4*)stats_ptrs[r]; cp.flag_peer[r] = (uint32_t*)flag_ptrs[r]; }
}

}  // namespace hippo

using namespace hippo;

// z: [C, V] fp32 logits of this rank's vocabulary shard; target: [C] local target index or -1.
extern "C" int hippo_ce_stats_push(const float* z, const long long* target, long long C, int V, void* const* stats_ptrs,
                                   void* const* flag_ptrs, int world, int rank, int max_rows, void* stream) {
  if (C <= 0) return 0;
  if (world < 1 || world > 8 || C > max_rows) return -2;
  CeCommParams cp; fill(cp, stats_ptrs, flag_ptrs, world, rank, max_rows, 0, 0);
  ce_stats_push_kernel<<<(unsigned)C, 512, 0, (cudaStream_t)stream>>>(z, target, V, cp);
  return (int)cudaGetLastError();
}

// part: [tiles_n][C] (max, sum exp) pairs and tz: [C] target logits from hippo_gemm_bf16_lce; target: [C] local target
// column or -1. Stores the merged triple of every row into slot [rank][row] of every rank's statistics buffer and
// releases C arrivals on every rank's counter [rank]. world == 1: stats_ptrs[0] is a local [max_rows] float4 buffer and
// flag_ptrs is not read.
extern "C" int hippo_ce_part_merge(const float* part, const float* tz, const long long* target, long long C, int tiles_n,
                                   void* const* stats_ptrs, void* const* flag_ptrs, int world, int rank, int max_rows,
                                   void* stream) {
  if (C <= 0) return 0;
  if (world < 1 || world > 8 || C > max_rows || tiles_n < 1) return -2;
  CeCommParams cp = {};
  cp.world = world; cp.rank = rank; cp.max_rows = max_rows; cp.wait_cycles = kWaitCycles;
  for (int r = 0; r < world; ++r) {
    cp.stats_peer[r] = (float4*)stats_ptrs[r];
    cp.flag_peer[r] = world > 1 ? (uint32_t*)flag_ptrs[r] : nullptr;
  }
  ce_part_merge_kernel<<<(unsigned)((C + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float2*)part, tz, target, C,
                                                                                       tiles_n, cp);
  return (int)cudaGetLastError();
}

// z: [C, V] bf16 logits (V a multiple of 8, rows contiguous), overwritten with dz. Other arguments as hippo_ce_grad_merge;
// world == 1 reads the local statistics buffer without waiting.
extern "C" int hippo_ce_grad_inplace(void* z, const long long* target, const float* roww, long long C, int V,
                                     float* loss_sum, void* const* stats_ptrs, void* const* flag_ptrs, int world, int rank,
                                     int max_rows, unsigned target_count, long long wait_cycles, void* stream) {
  if (C <= 0) return 0;
  if (world < 1 || world > 8 || C > max_rows || (V % 8) || ((uintptr_t)z & 15)) return -2;
  CeCommParams cp = {};
  cp.world = world; cp.rank = rank; cp.max_rows = max_rows; cp.target = target_count;
  cp.wait_cycles = wait_cycles > 0 ? wait_cycles : kWaitCycles;
  for (int r = 0; r < world; ++r) {
    cp.stats_peer[r] = (float4*)stats_ptrs[r];
    cp.flag_peer[r] = world > 1 ? (uint32_t*)flag_ptrs[r] : nullptr;
  }
  ce_grad_inplace_kernel<<<(unsigned)C, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)z, target, roww, V, loss_sum, cp);
  return (int)cudaGetLastError();
}

// dz: [C, V] bf16; roww: [C] row weight (valid / n_valid); loss_sum: device fp32[1], receives sum(lse - z_target) over
// rows with a positive weight. `target_count`: counter value that means all C rows of this call have arrived.
extern "C" int hippo_ce_grad_merge(const float* z, const long long* target, const float* roww, void* dz, long long C, int V,
                                   float* loss_sum, void* const* stats_ptrs, void* const* flag_ptrs, int world, int rank,
                                   int max_rows, unsigned target_count, long long wait_cycles, void* stream) {
  if (C <= 0) return 0;
  if (world < 1 || world > 8 || C > max_rows) return -2;
  CeCommParams cp; fill(cp, stats_ptrs, flag_ptrs, world, rank, max_rows, target_count, wait_cycles);
  ce_grad_merge_kernel<<<(unsigned)C, 512, 0, (cudaStream_t)stream>>>(z, target, roww, (__nv_bfloat16*)dz, V, loss_sum, cp);
  return (int)cudaGetLastError();
}
