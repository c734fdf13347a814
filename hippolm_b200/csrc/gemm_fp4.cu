// Block-scaled NVFP4 GEMM on the FP4 tensor cores:  C[M,N] = (A_fp4 * sfA) (B_fp4 * sfB)^T * gsA * gsB
//
//   tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X  (E2M1 data, one UE4M3 scale per 16
//   elements along K, MMA shape 128 x 128 x 64, fp32 accumulators in TMEM)
//
// A: [M, K/2] packed bytes (activations, quantised on the fly), B: [N, K/2] packed bytes (weights), both
// K-major. Scale factors arrive in the 512-byte "128 rows x 4 k-groups" tiles the MMA reads from TMEM
// (byte (m%32)*16 + ((m%128)/32)*4 + kgroup); a plain bulk copy brings one stage's tiles to shared memory
// and tcgen05.cp (32x128b.warpx4) moves each tile into 4 TMEM columns right before its MMA.
// Same persistent warp-specialised skeleton as the bf16 GEMM: TMA producer warp, single-thread MMA issuer,
// four epilogue warps, 128x128 tiles, K slabs of 256 elements (128 bytes, one swizzle atom), 5 stages,
// two TMEM accumulators. Replaces the reference's Marlin W4A16 path (bf16 mma.sync after dequant,
// src/models/ops/cuda/marlin_build/sources/marlin/marlin_template.h).
#include "sm100.cuh"
#include "host_utils.h"
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <stdlib.h>

namespace hippo {

constexpr int F_BM = 128, F_BN = 128, F_BKB = 128;          // K slab: 128 bytes = 256 fp4 elements = 4 MMAs
constexpr int F_STAGES = 5;
constexpr int F_A_BYTES = F_BM * F_BKB, F_B_BYTES = F_BN * F_BKB, F_SF_BYTES = 4 * 512;   // per operand per stage
constexpr int F_STAGE_BYTES = F_A_BYTES + F_B_BYTES + 2 * F_SF_BYTES;
constexpr int F_THREADS = 256;                              // TMA, MMA, 4 epilogue warps, 2 scale-copy warps
constexpr int F_SMEM = F_STAGES * F_STAGE_BYTES + 1024 + 256;
constexpr int F_RS_PITCH = 272;                             // slab row pitch: 16-byte stores of a quarter warp hit distinct banks
constexpr int F_RS_SLAB_BYTES = 4 * 32 * F_RS_PITCH;        // epilogue staging of the reduce-scatter variant
constexpr int F_SMEM_RS = F_SMEM + F_RS_SLAB_BYTES;
constexpr int F_TMEM_SF0 = 256;                             // accumulators use columns [0, 256)

struct Fp4Params {
  int M, N, K;                   // K in elements (multiple of 256)
  const uint8_t* sfa;            // tiled scales of A: [ceil(M/128)][K/64][512]
  const uint8_t* sfb;            // tiled scales of B: [ceil(N/128)][K/64][512]
  const float* gsa; const float* gsb;   // F_COMM_AG: gsa points at one tensor scale per source rank
  __nv_bfloat16* C; long long ldc;
  int accumulate;                // plain mode: C += result (the weight-gradient product adds into the accumulator)
  int tiles_m, tiles_n;
  // F_COMM_AG: A (packed bytes, scale tiles, per-source tensor scales) is this rank's gathered FP4 buffer, filled
  // shard by shard by every rank's nvfp4_quant_push_kernel; `flags[src * (rows_per_shard/128) + row block]`
  // reaches `target` once all K slabs of that row block have landed.
  int world, rank, rows_per_shard;
  const uint32_t* flags; uint32_t target; long long wait_cycles;
  // F_COMM_RS: partial tiles go to the staging slot [rank] of the rank that owns the rows, then every rank sums its slots
  void* stage_peer[8]; uint32_t* rs_flag_peer[8]; uint32_t rs_target; void* out_local;
};

constexpr int F_COMM_NONE = 0, F_COMM_AG = 1, F_COMM_RS = 2;

__device__ __forceinline__ uint32_t f_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float f_ld_relaxed_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void f_red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded spin on a monotonic counter written by other GPUs
__device__ __forceinline__ bool f_wait_counter(const uint32_t* p, uint32_t target, long long limit, int detail) {
  if ((int32_t)(f_ld_acquire_sys(p) - target) >= 0) return true;
  long long t0 = clock64();
  while ((int32_t)(f_ld_acquire_sys(p) - target) < 0) {
    if (clock64() - t0 > limit) { report(kWaitPeerFlag, detail); return false; }
    __nanosleep(64);
  }
  return true;
}

__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int COMM>
__global__ void __launch_bounds__(F_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ Fp4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* epi_stage = smem + F_STAGES * F_STAGE_BYTES;      // F_COMM_RS only: 4 warps x [32 rows][256 B]
  uint64_t* full = (uint64_t*)(smem + F_STAGES * F_STAGE_BYTES + (COMM == F_COMM_RS ? F_RS_SLAB_BYTES : 0));
  uint64_t* empty = full + F_STAGES;
  uint64_t* tfull = empty + F_STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* sf_full = tempty + 2;                              // scale tiles of a stage are in TMEM (2 copy warps)
  uint32_t* tmem_slot = (uint32_t*)(sf_full + F_STAGES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = p.K / 256;
  const int k64 = p.K / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&sf_full[s], 2); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // grouped rasterisation; with a fused collective the row blocks are walked shard by shard: all-gather in arrival
  // order (own, rank-1, rank-2, ...), reduce-scatter remote owners first (rank+1, ...), own rows last
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int GROUP = 8;
    int tiles_m = p.tiles_m, base_m = 0;
    if (COMM != F_COMM_NONE) {
      const int tms = p.rows_per_shard / F_BM;
      const int per_shard = tms * p.tiles_n;
      const int si = t / per_shard;
      t -= si * per_shard;
      const int shard = (COMM == F_COMM_AG) ? (p.rank - si + p.world) % p.world : (p.rank + 1 + si) % p.world;
      base_m = shard * tms; tiles_m = tms;
    }
    int per_group = GROUP * p.tiles_n;
    int g = t / per_group, r = t % per_group;
    int gm = min(GROUP, tiles_m - g * GROUP);
    tm = base_m + g * GROUP + r % gm;
    tn = r / gm;
  };

  if (warp == 0) {
    if (lane == 0) {
      int it = 0; bool ok = true;
      int last_tm = -1;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn; tile_coord(t, tm, tn);
        if (COMM == F_COMM_AG && tm != last_tm) {
          const int bps = p.rows_per_shard / F_BM;
          if (tm / bps != p.rank) {                          // own rows were written by the previous local kernel
            ok = f_wait_counter(p.flags + tm, p.target, p.wait_cycles, tm);
            asm volatile("fence.proxy.async;" ::: "memory");  // remote generic-proxy writes -> TMA / bulk reads
            if (!ok) break;
          }
          last_tm = tm;
        }
        for (int kb = 0; kb < kblocks && ok; ++kb, ++it) {
          int s = it % F_STAGES; uint32_t ph = (it / F_STAGES) & 1;
          ok = mbar_wait(&empty[s], ph ^ 1, kWaitSmemEmpty, it);
          if (!ok) break;
          uint8_t* sa = smem + s * F_STAGE_BYTES; uint8_t* sb = sa + F_A_BYTES;
          uint8_t* ssa = sb + F_B_BYTES; uint8_t* ssb = ssa + F_SF_BYTES;
          mbar_expect_tx(&full[s], F_STAGE_BYTES);
          tma_load_2d(sa, &tmA, &full[s], kb * F_BKB, tm * F_BM);
          tma_load_2d(sb, &tmB, &full[s], kb * F_BKB, tn * F_BN);
          bulk_copy_g2s(ssa, p.sfa + ((long long)tm * k64 + kb * 4) * 512, F_SF_BYTES, &full[s]);
          bulk_copy_g2s(ssb, p.sfb + ((long long)tn * k64 + kb * 4) * 512, F_SF_BYTES, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_nvf4(F_BM, F_BN);
      int it = 0, tl = 0; bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tl) {
        int acc = tl & 1; uint32_t aph = (tl >> 1) & 1;
        ok = mbar_wait(&tempty[acc], aph ^ 1, kWaitTmemEmpty, tl);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * F_BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          int s = it % F_STAGES; uint32_t ph = (it / F_STAGES) & 1;
          ok = mbar_wait(&sf_full[s], ph, kWaitTmaFull, it);   // operands landed and the stage's scales are in TMEM
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * F_STAGE_BYTES), sb = sa + F_A_BYTES;
          const uint32_t t_sf = tmem_base + F_TMEM_SF0 + s * 32;          // 16 columns SFA + 16 columns SFB
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint64_t ad = make_smem_desc(sa + k * 32, 16, 1024);
            uint64_t bd = make_smem_desc(sb + k * 32, 16, 1024);
            mma_nvf4_ss(d_tmem, ad, bd, idesc, t_sf + k * 4, t_sf + 16 + k * 4, (kb | k) ? 1u : 0u);
          }
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&tfull[acc]);
      }
    }
  } else if (warp >= 6) {
    // Scale-copy warps: one thread cannot issue a slab's 8 tcgen05.cp, 4 MMAs and the commit as fast as the tensor pipe
    // retires the MMAs, so the copies (warp 6: the A tiles, warp 7: the B tiles) have their own threads, each
    // committing to the stage's sf_full barrier; the stage's 32 scale columns are free again once its previous MMAs
    // have completed, which the producer has seen before it refilled the stage.
    if (lane == 0) {
      const int part = warp - 6;
      const int my_tiles = (int)blockIdx.x < num_tiles ? (num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
      const int total_its = my_tiles * kblocks;
      for (int it = 0; it < total_its; ++it) {
        const int s = it % F_STAGES; const uint32_t ph = (it / F_STAGES) & 1;
        if (!mbar_wait(&full[s], ph, kWaitTmaFull, it)) break;
        tc_fence_after();
        const uint32_t src = smem_u32(smem + s * F_STAGE_BYTES) + F_A_BYTES + F_B_BYTES + part * F_SF_BYTES;
        const uint32_t t_sf = tmem_base + F_TMEM_SF0 + s * 32 + part * 16;
#pragma unroll
        for (int k = 0; k < 4; ++k)   // 32 rows x 16 bytes, rows contiguous: 8-row groups are 128 bytes apart, no swizzle
          tc_cp_32x128b_warpx4(t_sf + k * 4, make_smem_desc_noswizzle(src + k * 512, 16, 128));
        tc_commit(&sf_full[s]);
      }
    }
  } else {
    const int q = warp & 3;
    int tl = 0; bool ok = true;
    int rs_pending = 0;                     // F_COMM_RS: tiles of the current owner shard stored but not yet released
    float alpha = (COMM == F_COMM_AG) ? 0.f : (*p.gsa) * (*p.gsb);
    const float gsb = *p.gsb;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tl) {
      int tm, tn; tile_coord(t, tm, tn);
      int acc = tl & 1; uint32_t aph = (tl >> 1) & 1;
      ok = mbar_wait(&tfull[acc], aph, kWaitTmemFull, tl);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      // the tensor scale of the source shard was pushed before the row block's counter was released
      if (COMM == F_COMM_AG) alpha = f_ld_relaxed_sys_f32(p.gsa + (tm * F_BM) / p.rows_per_shard) * gsb;
      const int row = tm * F_BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * F_BN + ((uint32_t)(q * 32) << 16);
      if (COMM == F_COMM_RS) {
        // The warp lays its 32 x 128 slab out in shared memory and every lane sends its own row (256 contiguous bytes) to
        // the owner's staging slot [this rank] with one bulk async copy, so the remote stores are in flight while the
        // warp drains the next tile.
        uint8_t* slab = epi_stage + (warp - 2) * 32 * F_RS_PITCH;
        tma_store_wait_read<0>();                                          // the previous tile's rows have left the slab
        __syncwarp();
#pragma unroll 1
        for (int c = 0; c < F_BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            __nv_bfloat162* vb = (__nv_bfloat162*)&v;
#pragma unroll
            for (int e = 0; e < 4; ++e)
              vb[e] = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * e]) * alpha, __uint_as_float(r[j + 2 * e + 1]) * alpha);
            *(uint4*)(slab + lane * F_RS_PITCH + (c + j) * 2) = v;
          }
        }
        fence_proxy_async();                                               // generic-proxy slab writes -> bulk copy reads
        const int row_base = tm * F_BM + q * 32;
        const int owner = row_base / p.rows_per_shard;
        const int ncols = min(F_BN, p.N - tn * F_BN);
        if (row_base + lane < p.M) {
          __nv_bfloat16* dst = (__nv_bfloat16*)p.stage_peer[owner] +
                               ((long long)p.rank * p.rows_per_shard + (row_base + lane - owner * p.rows_per_shard)) * p.N + tn * F_BN;
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                       ::"l"(dst), "r"(smem_u32(slab + lane * F_RS_PITCH)), "r"((uint32_t)(ncols * 2)) : "memory");
        }
        tma_store_commit();
        // one completion wait + counter release per OWNER SHARD (the owner reduces only after a source's last tile anyway)
        ++rs_pending;
        const int tnext = t + (int)gridDim.x;
        int owner_next = -1;
        if (tnext < num_tiles) { int tm2, tn2; tile_coord(tnext, tm2, tn2); owner_next = (tm2 * F_BM + q * 32) / p.rows_per_shard; }
        if (owner_next != owner) {
          tma_store_wait<0>();                                             // this lane's rows have landed
          __threadfence_system();
          __syncwarp();
          if (lane == 0) f_red_release_sys_add(p.rs_flag_peer[owner] + p.rank, (uint32_t)rs_pending);
          rs_pending = 0;
        }
      } else
#pragma unroll 1
      for (int c = 0; c < F_BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tc_wait_ld();
        const int col0 = tn * F_BN + c;
        if (row < p.M && col0 < p.N) {
          __nv_bfloat16* crow = p.C + (long long)row * p.ldc + col0;
          if (col0 + 32 <= p.N) {
            uint4 old[4];
            if (p.accumulate) {
#pragma unroll
              for (int j = 0; j < 4; ++j) old[j] = *(const uint4*)(crow + 8 * j);   // four loads in flight
            }
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v;
              __nv_bfloat162* vb = (__nv_bfloat162*)&v;
              const __nv_bfloat162* ob = (const __nv_bfloat162*)&old[j / 8];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float lo = __uint_as_float(r[j + 2 * e]) * alpha, hi = __uint_as_float(r[j + 2 * e + 1]) * alpha;
                if (p.accumulate) { const float2 o2 = __bfloat1622float2(ob[e]); lo += o2.x; hi += o2.y; }
                vb[e] = __floats2bfloat162_rn(lo, hi);
              }
              *(uint4*)(crow + j) = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) {
                float v = __uint_as_float(r[j]) * alpha;
                if (p.accumulate) v += __bfloat162float(crow[j]);
                crow[j] = __float2bfloat16(v);
              }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
  if (COMM == F_COMM_RS) {
    // reduction of the rows this rank owns: wait (bounded) for every source, then sum the staging slots
    if ((int)threadIdx.x < p.world)
      f_wait_counter(p.rs_flag_peer[p.rank] + threadIdx.x, p.rs_target, p.wait_cycles, 100 + threadIdx.x);
    __syncthreads();
    const long long nvec = (long long)p.rows_per_shard * p.N / 8;
    const uint4* stage = (const uint4*)p.stage_peer[p.rank];
    uint4* out = (uint4*)p.out_local;
    const long long stride = (long long)gridDim.x * F_THREADS;
    for (long long v0 = (long long)blockIdx.x * F_THREADS + threadIdx.x; v0 < nvec; v0 += stride * 4) {
      float acc[4][8];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
      for (int sidx = 0; sidx < p.world; ++sidx) {
        uint4 x[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long v = v0 + j * stride;
          x[j] = v < nvec ? __ldcg(stage + (long long)sidx * nvec + v) : make_uint4(0, 0, 0, 0);   // written by another GPU: bypass L1
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162* xb = (const __nv_bfloat162*)&x[j];
#pragma unroll
          for (int e = 0; e < 4; ++e) { float2 f = __bfloat1622float2(xb[e]); acc[j][2 * e] += f.x; acc[j][2 * e + 1] += f.y; }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long v = v0 + j * stride;
        if (v < nvec) {
          uint4 o;
          __nv_bfloat162* ob = (__nv_bfloat162*)&o;
#pragma unroll
          for (int e = 0; e < 4; ++e) ob[e] = __floats2bfloat162_rn(acc[j][2 * e], acc[j][2 * e + 1]);
          out[v] = o;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Quantise this rank's activation shard x[rows, K] (bf16) to NVFP4 and push the result straight into every rank's
// gathered buffer (own rank included): packed bytes at row offset rank*rows, scale bytes already in the 512-byte
// MMA tile layout, and the shard's tensor scale at slot [rank]. One CTA per (128-row block, 512-column slab): the
// slab is quantised into shared memory first so that every remote store is a full 16-byte vector, then the CTA
// releases the (source rank, row block) arrival counter on each destination. The all-gather therefore moves
// 0.5625 bytes per element instead of 2, and the consumer GEMM (F_COMM_AG) starts on whatever has arrived.
// Buffer layout on every rank: [T, K/2] packed | [T/128][K/64][512] scale tiles | 8 x fp32 tensor scales.
struct QuantPushParams {
  const __nv_bfloat16* x; long long ldx; int rows, K;
  const float* gs;                 // this shard's tensor scale (device fp32[1])
  int world, rank;
  uint8_t* buf_peer[8];
  uint32_t* flag_peer[8];
};

__global__ void __launch_bounds__(256)
nvfp4_quant_push_kernel(const __grid_constant__ QuantPushParams q) {
  __shared__ __align__(16) uint8_t s_packed[128 * 256];
  __shared__ __align__(16) uint8_t s_sf[8 * 512];
  const int tid = threadIdx.x;
  const int k0 = blockIdx.x * 512, rb = blockIdx.y, row0 = rb * 128;
  const float gs = *q.gs;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int blk = tid + i * 256, r = blk >> 5, kb = blk & 31;
    const __nv_bfloat16* src = q.x + (long long)(row0 + r) * q.ldx + k0 + kb * 16;
    uint4 raw[2] = {__ldg((const uint4*)src), __ldg((const uint4*)src + 1)};
    const __nv_bfloat162* h2 = (const __nv_bfloat162*)raw;
    float f[16];
#pragma unroll
    for (int e = 0; e < 8; ++e) { float2 t = __bfloat1622float2(h2[e]); f[2 * e] = t.x; f[2 * e + 1] = t.y; }
    float bm = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) bm = fmaxf(bm, fabsf(f[e]));
    const float sraw = fminf(bm / 6.f / gs, 448.f);
    const __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(sraw, __NV_SATFINITE, __NV_E4M3);
    const float sdec = __half2float(__half(__nv_cvt_fp8_to_halfraw(s8, __NV_E4M3))) * gs;
    uint2 outv;
    uint8_t* ob = (uint8_t*)&outv;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      // division (not reciprocal multiply) keeps ties identical to the stand-alone quantise kernel
      const float lo = sdec > 0.f ? f[2 * e] / sdec : f[2 * e], hi = sdec > 0.f ? f[2 * e + 1] / sdec : f[2 * e + 1];
      ob[e] = (uint8_t)__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
    }
    *(uint2*)(s_packed + r * 256 + kb * 8) = outv;
    s_sf[(kb >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = (uint8_t)s8;
  }
  __syncthreads();
  const long long T = (long long)q.world * q.rows;
  const long long sf_off = T * (q.K / 2), gs_off = sf_off + T * (q.K / 16);
  const int bps = q.rows / 128;
  for (int d = 0; d < q.world; ++d) {
    const int peer = (q.rank + d) % q.world;
    uint8_t* base = q.buf_peer[peer];
    uint8_t* pk = base + ((long long)q.rank * q.rows + row0) * (q.K / 2) + k0 / 2;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int v = tid + j * 256, r = v >> 4, c = v & 15;
      *(uint4*)(pk + (long long)r * (q.K / 2) + c * 16) = *(const uint4*)(s_packed + r * 256 + c * 16);
    }
    uint8_t* sf = base + sf_off + (((long long)q.rank * q.rows + row0) / 128 * (q.K / 64) + k0 / 64) * 512;
    *(uint4*)(sf + tid * 16) = *(const uint4*)(s_sf + tid * 16);
    if (tid == 0) ((float*)(base + gs_off))[q.rank] = gs;
    __threadfence_system();
    __syncthreads();
    if (tid == 0) f_red_release_sys_add(q.flag_peer[peer] + q.rank * bps + rb, 1u);
  }
}

// Transposed NVFP4 quantisation for the weight-gradient product dW = dY^T x, whose contraction runs over TOKENS:
// x[T, C] (bf16, row pitch ldx) -> packed [C, T/2] (16-element blocks along T), block scales written straight into the
// 512-byte MMA tile layout [ceil(C/128)][T/64][512] (no separate re-tiling pass). One CTA transposes a 256-token x
// 64-channel tile through shared memory: coalesced 128-byte row reads, then thread (channel, 64-token group) quantises
// four 16-token blocks and writes 32 contiguous packed bytes and 4 contiguous scale bytes.
__global__ void __launch_bounds__(256)
nvfp4_quant_transposed_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, long long T, int C, const float* gs_ptr,
                              uint8_t* __restrict__ packed, uint8_t* __restrict__ sf_tiled) {
  __shared__ __nv_bfloat16 tile[256][66];
  const long long t0 = (long long)blockIdx.x * 256;
  const int c0 = blockIdx.y * 64;
  const int tid = threadIdx.x;
  // 256 rows x 64 channels = 2048 16-byte vectors; rows beyond T or channels beyond C read as zero
  for (int v = tid; v < 2048; v += 256) {
    const int r = v >> 3, cv = (v & 7) * 8;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (t0 + r < T && c0 + cv < C) val = __ldg((const uint4*)(x + (t0 + r) * ldx + c0 + cv));
    const __nv_bfloat162* h = (const __nv_bfloat162*)&val;
#pragma unroll
    for (int e = 0; e < 4; ++e) *(__nv_bfloat162*)&tile[r][cv + 2 * e] = h[e];
  }
  __syncthreads();
  const int c = tid & 63, q = tid >> 6;                      // channel, group of four 16-token blocks
  if (c0 + c >= C) return;
  const float gs = *gs_ptr;
  const long long kg0 = t0 / 16 + q * 4;                     // first k-group (16-token block) of this thread
  uint4 outv[2];
  uint8_t* ob = (uint8_t*)outv;
  uint32_t sfw = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    float f[16], bm = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) { f[e] = __bfloat162float(tile[q * 64 + b * 16 + e][c]); bm = fmaxf(bm, fabsf(f[e])); }
    const float sraw = fminf(bm / 6.f / gs, 448.f);
    const __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(sraw, __NV_SATFINITE, __NV_E4M3);
    const float sdec = __half2float(__half(__nv_cvt_fp8_to_halfraw(s8, __NV_E4M3))) * gs;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float lo = sdec > 0.f ? f[2 * e] / sdec : f[2 * e], hi = sdec > 0.f ? f[2 * e + 1] / sdec : f[2 * e + 1];
      ob[b * 8 + e] = (uint8_t)__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
    }
    sfw |= (uint32_t)s8 << (8 * b);
  }
  const long long tq = t0 + q * 64;
  if (tq < T) {                                              // T is a multiple of 64 (checked by the launcher)
    const int m = c0 + c;
    uint4* dst = (uint4*)(packed + (long long)m * (T / 2) + tq / 2);
    dst[0] = outv[0]; dst[1] = outv[1];
    const long long tile_idx = (long long)(m / 128) * (T / 64) + kg0 / 4;
    *(uint32_t*)(sf_tiled + tile_idx * 512 + (m % 32) * 16 + ((m % 128) / 32) * 4) = sfw;
  }
}

// logical e4m3 scales [rows, K/16] -> 512-byte tiles [ceil(rows/128)][K/64][(m%32)*16 + ((m%128)/32)*4 + kg]
__global__ void nvfp4_tile_scales_kernel(const uint8_t* __restrict__ sf, uint8_t* __restrict__ out, long long rows,
                                         int kgroups /* K/16 */, long long rows_padded) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = rows_padded * kgroups;
  if (idx >= total) return;
  long long m = idx / kgroups; int kg = (int)(idx % kgroups);
  uint8_t v = m < rows ? sf[m * kgroups + kg] : (uint8_t)0;
  long long tile = (m / 128) * (kgroups / 4) + kg / 4;
  out[tile * 512 + (m % 32) * 16 + ((m % 128) / 32) * 4 + (kg % 4)] = v;
}

}  // namespace hippo

using namespace hippo;

static thread_local int g_fp4_accumulate = 0;   // set by hippo_gemm_nvfp4_accumulate for the next plain launch

extern "C" int hippo_nvfp4_tile_scales(const void* sf, void* out, long long rows, long long K, void* stream) {
  if (K % 64) return -1;
  long long rp = (rows + 127) / 128 * 128;
  long long total = rp * (K / 16);
  nvfp4_tile_scales_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)sf, (uint8_t*)out, rows, (int)(K / 16), rp);
  return (int)cudaGetLastError();
}

extern "C" int hippo_gemm_nvfp4_pair(const void* A, const void* B, const void* sfa, const void* sfb, const float* gsa,
                                     const float* gsb, void* C, int M, int N, int K, long long ldc, int accumulate,
                                     void* stream);
extern "C" int hippo_allgather_gemm_nvfp4_pair(const void* gathered, const void* flags, int world, int rank,
                                               int rows_per_shard, const void* B, const void* sfb, const float* gsb,
                                               void* C, long long ldc, int N, int K, unsigned target,
                                               long long wait_cycles, void* stream);
extern "C" int hippo_gemm_reduce_scatter_nvfp4_pair(const void* A, const void* sfa, const float* gsa, const void* B,
                                                    const void* sfb, const float* gsb, void* const* stage_ptrs,
                                                    void* const* flag_ptrs, int world, int rank, int rows_per_shard,
                                                    void* out_local, int N, int K, unsigned target,
                                                    long long wait_cycles, void* stream);

// Products with at least 256 rows and columns run on the CTA-pair kernel of gemm_fp4_2sm.cu (HIPPO_FP4_PAIR=0: never).
static int fp4_pair_mode() {
  static int mode = -1;
  if (mode < 0) { const char* e = getenv("HIPPO_FP4_PAIR"); mode = e ? atoi(e) : 1; }
  return mode;
}

// A: [M, K/2] packed fp4 bytes, B: [N, K/2]; sfa/sfb: tiled scales (hippo_nvfp4_tile_scales); gsa/gsb: device fp32[1].
extern "C" int hippo_gemm_nvfp4(const void* A, const void* B, const void* sfa, const void* sfb, const float* gsa,
                                const float* gsb, void* C, int M, int N, int K, long long ldc, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 256 || (N % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)C & 15) || (ldc % 8)) return -2;
  if (fp4_pair_mode() && M >= 256 && N >= 256) {
    const int acc = g_fp4_accumulate;
    g_fp4_accumulate = 0;
    return hippo_gemm_nvfp4_pair(A, B, sfa, sfb, gsa, gsb, C, M, N, K, ldc, acc, stream);
  }
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, (uint64_t)K / 2, (uint64_t)M, (uint64_t)K / 2, F_BKB, F_BM, 1, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, F_BKB, F_BN, 1, true);
  if (rc) return rc;
  Fp4Params p;
  p.M = M; p.N = N; p.K = K; p.sfa = (const uint8_t*)sfa; p.sfb = (const uint8_t*)sfb; p.gsa = gsa; p.gsb = gsb;
  p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.accumulate = g_fp4_accumulate; g_fp4_accumulate = 0;
  p.tiles_m = (M + F_BM - 1) / F_BM; p.tiles_n = (N + F_BN - 1) / F_BN;
  int tiles = p.tiles_m * p.tiles_n, sms = sm_count();
  int grid = tiles < sms ? tiles : sms;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel<F_COMM_NONE>, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  gemm_nvfp4_kernel<F_COMM_NONE><<<grid, F_THREADS, F_SMEM, (cudaStream_t)stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}

// Same product, added into C (bf16): C += (A sfa)(B sfb)^T gsa gsb.
extern "C" int hippo_gemm_nvfp4_accumulate(const void* A, const void* B, const void* sfa, const void* sfb, const float* gsa,
                                           const float* gsb, void* C, int M, int N, int K, long long ldc, void* stream) {
  g_fp4_accumulate = 1;
  return hippo_gemm_nvfp4(A, B, sfa, sfb, gsa, gsb, C, M, N, K, ldc, stream);
}

// x[T, C] bf16 -> NVFP4 of x^T: packed [C, T/2], scales in MMA tile layout [ceil(C/128)][T/64][512] (zero-filled by the
// caller when C is not a multiple of 128), against the tensor scale *gs. T must be a multiple of 64, C of 8.
extern "C" int hippo_nvfp4_quantize_transposed(const void* x, long long ldx, long long T, int C, const float* gs,
                                               void* packed, void* sf_tiled, void* stream) {
  if (T <= 0 || C <= 0) return 0;
  if ((T % 64) || (C % 8) || (ldx % 8) || ((uintptr_t)x & 15) || ((uintptr_t)packed & 15)) return -2;
  dim3 grid((unsigned)((T + 255) / 256), (unsigned)((C + 63) / 64));
  nvfp4_quant_transposed_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ldx, T, C, gs,
                                                                       (uint8_t*)packed, (uint8_t*)sf_tiled);
  return (int)cudaGetLastError();
}

// Gathered FP4 buffer (layout above) -> bf16 [T, K]: the activations exactly as the FP4 GEMM consumed them,
// for the weight-gradient product of the backward pass. One thread per 16-element block.
__global__ void nvfp4_dequant_gathered_kernel(const uint8_t* __restrict__ buf, long long T, int K, int rows_per_shard,
                                              __nv_bfloat16* __restrict__ out) {
  const long long nb = T * (K / 16);
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= nb) return;
  const long long m = b / (K / 16);
  const int kg = (int)(b % (K / 16));
  const long long sf_off = T * (K / 2), gs_off = sf_off + T * (K / 16);
  const float gs = ((const float*)(buf + gs_off))[m / rows_per_shard];
  const uint8_t s8 = buf[sf_off + ((m / 128) * (K / 64) + kg / 4) * 512 + (m % 32) * 16 + ((m % 128) / 32) * 4 + (kg % 4)];
  const float sc = __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)s8, __NV_E4M3))) * gs;
  const float lut[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const uint2 pv = *(const uint2*)(buf + b * 8);
  const uint8_t* pb = (const uint8_t*)&pv;
  uint4 o[2];
  __nv_bfloat162* ob = (__nv_bfloat162*)o;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint8_t lo = pb[i] & 0xF, hi = pb[i] >> 4;
    ob[i] = __floats2bfloat162_rn(((lo & 8) ? -lut[lo & 7] : lut[lo & 7]) * sc, ((hi & 8) ? -lut[hi & 7] : lut[hi & 7]) * sc);
  }
  uint4* dst = (uint4*)(out + b * 16);
  dst[0] = o[0]; dst[1] = o[1];
}

extern "C" int hippo_nvfp4_dequant_gathered(const void* buf, long long T, int K, int rows_per_shard, void* out, void* stream) {
  if (T <= 0 || K % 64 || rows_per_shard <= 0 || (T % 128)) return -2;
  const long long nb = T * (K / 16);
  nvfp4_dequant_gathered_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)buf, T, K, rows_per_shard, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}

// Quantise + push (see nvfp4_quant_push_kernel). x: [rows, K] bf16 with pitch ldx; rows % 128 == 0, K % 512 == 0.
// buf_ptrs[r] / flag_ptrs[r]: rank r's gathered FP4 buffer and its arrival counters [world * rows/128].
extern "C" int hippo_nvfp4_quant_push(const void* x, long long ldx, int rows, int K, const float* gs,
                                      void* const* buf_ptrs, void* const* flag_ptrs, int world, int rank, void* stream) {
  if (rows <= 0 || rows % 128 || K % 512 || world < 1 || world > 8 || ((uintptr_t)x & 15) || (ldx % 8)) return -2;
  QuantPushParams q;
  q.x = (const __nv_bfloat16*)x; q.ldx = ldx; q.rows = rows; q.K = K; q.gs = gs; q.world = world; q.rank = rank;
  for (int r = 0; r < world; ++r) { q.buf_peer[r] = (uint8_t*)buf_ptrs[r]; q.flag_peer[r] = (uint32_t*)flag_ptrs[r]; }
  nvfp4_quant_push_kernel<<<dim3(K / 512, rows / 128), 256, 0, (cudaStream_t)stream>>>(q);
  return (int)cudaGetLastError();
}

// All-gather -> FP4 GEMM, consumer side: C[world*rows_per_shard, N] = gathered(A) * B^T. `gathered` is this rank's
// gathered FP4 buffer (layout in nvfp4_quant_push_kernel), `flags` its arrival counters, `target` the counter value
// that means "this call's slabs have all landed" (calls so far * K/512).
extern "C" int hippo_allgather_gemm_nvfp4(const void* gathered, const void* flags, int world, int rank,
                                          int rows_per_shard, const void* B, const void* sfb, const float* gsb, void* C,
                                          long long ldc, int N, int K, unsigned target, long long wait_cycles,
                                          void* stream) {
  if (world < 1 || world > 8 || rows_per_shard % F_BM || K % 512 || (N % 8) || (ldc % 8)) return -2;
  if (fp4_pair_mode() && rows_per_shard % 256 == 0 && N >= 256)
    return hippo_allgather_gemm_nvfp4_pair(gathered, flags, world, rank, rows_per_shard, B, sfb, gsb, C, ldc, N, K, target,
                                           wait_cycles, stream);
  const int M = world * rows_per_shard;
  const uint8_t* base = (const uint8_t*)gathered;
  const long long sf_off = (long long)M * (K / 2), gs_off = sf_off + (long long)M * (K / 16);
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, base, (uint64_t)K / 2, (uint64_t)M, (uint64_t)K / 2, F_BKB, F_BM, 1, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, F_BKB, F_BN, 1, true);
  if (rc) return rc;
  Fp4Params p = {};
  p.M = M; p.N = N; p.K = K; p.sfa = base + sf_off; p.sfb = (const uint8_t*)sfb;
  p.gsa = (const float*)(base + gs_off); p.gsb = gsb; p.C = (__nv_bfloat16*)C; p.ldc = ldc;
  p.tiles_m = M / F_BM; p.tiles_n = (N + F_BN - 1) / F_BN;
  p.world = world; p.rank = rank; p.rows_per_shard = rows_per_shard;
  p.flags = (const uint32_t*)flags; p.target = target; p.wait_cycles = wait_cycles > 0 ? wait_cycles : kWaitCycles;
  int tiles = p.tiles_m * p.tiles_n, sms = sm_count();
  int grid = tiles < sms ? tiles : sms;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel<F_COMM_AG>, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  gemm_nvfp4_kernel<F_COMM_AG><<<grid, F_THREADS, F_SMEM, (cudaStream_t)stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}

// FP4 GEMM -> reduce-scatter. A: [world*rows_per_shard, K/2] local packed activations (+ tiled scales, tensor scale);
// partial C tiles go to the staging slot [rank] of the owning rank (stage_ptrs[r]: [world][rows_per_shard, N] bf16 on
// rank r); every rank then sums its slots into out_local [rows_per_shard, N].
// `target` = calls so far * (rows_per_shard/128) * ceil(N/128) * 4.
extern "C" int hippo_gemm_reduce_scatter_nvfp4(const void* A, const void* sfa, const float* gsa, const void* B,
                                               const void* sfb, const float* gsb, void* const* stage_ptrs,
                                               void* const* flag_ptrs, int world, int rank, int rows_per_shard,
                                               void* out_local, int N, int K, unsigned target, long long wait_cycles,
                                               void* stream) {
  if (world < 1 || world > 8 || rows_per_shard % F_BM || K % 256 || (N % 8)) return -2;
  if (fp4_pair_mode() && rows_per_shard % 256 == 0 && N >= 256)
    return hippo_gemm_reduce_scatter_nvfp4_pair(A, sfa, gsa, B, sfb, gsb, stage_ptrs, flag_ptrs, world, rank, rows_per_shard,
                                                out_local, N, K, target, wait_cycles, stream);
  const int M = world * rows_per_shard;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, (uint64_t)K / 2, (uint64_t)M, (uint64_t)K / 2, F_BKB, F_BM, 1, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, F_BKB, F_BN, 1, true);
  if (rc) return rc;
  Fp4Params p = {};
  p.M = M; p.N = N; p.K = K; p.sfa = (const uint8_t*)sfa; p.sfb = (const uint8_t*)sfb; p.gsa = gsa; p.gsb = gsb;
  p.C = nullptr; p.ldc = N;
  p.tiles_m = M / F_BM; p.tiles_n = (N + F_BN - 1) / F_BN;
  p.world = world; p.rank = rank; p.rows_per_shard = rows_per_shard;
  p.wait_cycles = wait_cycles > 0 ? wait_cycles : kWaitCycles;
  for (int r = 0; r < world; ++r) { p.stage_peer[r] = stage_ptrs[r]; p.rs_flag_peer[r] = (uint32_t*)flag_ptrs[r]; }
  p.rs_target = target; p.out_local = out_local;
  int tiles = p.tiles_m * p.tiles_n, sms = sm_count();
  int grid = tiles < sms ? tiles : sms;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel<F_COMM_RS>, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM_RS);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  gemm_nvfp4_kernel<F_COMM_RS><<<grid, F_THREADS, F_SMEM_RS, (cudaStream_t)stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}
