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

namespace hippo {

constexpr int F_BM = 128, F_BN = 128, F_BKB = 128;          // K slab: 128 bytes = 256 fp4 elements = 4 MMAs
constexpr int F_STAGES = 5;
constexpr int F_A_BYTES = F_BM * F_BKB, F_B_BYTES = F_BN * F_BKB, F_SF_BYTES = 4 * 512;   // per operand per stage
constexpr int F_STAGE_BYTES = F_A_BYTES + F_B_BYTES + 2 * F_SF_BYTES;
constexpr int F_THREADS = 192;
constexpr int F_SMEM = F_STAGES * F_STAGE_BYTES + 1024 + 256;
constexpr int F_TMEM_SF0 = 256;                             // accumulators use columns [0, 256)

struct Fp4Params {
  int M, N, K;                   // K in elements (multiple of 256)
  const uint8_t* sfa;            // tiled scales of A: [ceil(M/128)][K/64][512]
  const uint8_t* sfb;            // tiled scales of B: [ceil(N/128)][K/64][512]
  const float* gsa; const float* gsb;
  __nv_bfloat16* C; long long ldc;
  int tiles_m, tiles_n;
};

__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(F_THREADS, 1)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Fp4Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + F_STAGES * F_STAGE_BYTES);
  uint64_t* empty = full + F_STAGES;
  uint64_t* tfull = empty + F_STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = (uint32_t*)(tempty + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = p.K / 256;
  const int k64 = p.K / 64;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int GROUP = 8;
    int per_group = GROUP * p.tiles_n;
    int g = t / per_group, r = t % per_group;
    int gm = min(GROUP, p.tiles_m - g * GROUP);
    tm = g * GROUP + r % gm;
    tn = r / gm;
  };

  if (warp == 0) {
    if (lane == 0) {
      int it = 0; bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn; tile_coord(t, tm, tn);
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
          ok = mbar_wait(&full[s], ph, kWaitTmaFull, it);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * F_STAGE_BYTES), sb = sa + F_A_BYTES;
          const uint32_t ssa = sb + F_B_BYTES, ssb = ssa + F_SF_BYTES;
          const uint32_t t_sf = tmem_base + F_TMEM_SF0 + s * 32;          // 16 columns SFA + 16 columns SFB
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // 32 rows x 16 bytes, rows contiguous: 8-row groups are 128 bytes apart, no swizzle
            tc_cp_32x128b_warpx4(t_sf + k * 4, make_smem_desc_noswizzle(ssa + k * 512, 16, 128));
            tc_cp_32x128b_warpx4(t_sf + 16 + k * 4, make_smem_desc_noswizzle(ssb + k * 512, 16, 128));
          }
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
  } else {
    const int q = warp & 3;
    int tl = 0; bool ok = true;
    const float alpha = (*p.gsa) * (*p.gsb);
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tl) {
      int tm, tn; tile_coord(t, tm, tn);
      int acc = tl & 1; uint32_t aph = (tl >> 1) & 1;
      ok = mbar_wait(&tfull[acc], aph, kWaitTmemFull, tl);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = tm * F_BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * F_BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < F_BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tc_wait_ld();
        const int col0 = tn * F_BN + c;
        if (row < p.M && col0 < p.N) {
          __nv_bfloat16* crow = p.C + (long long)row * p.ldc + col0;
          if (col0 + 32 <= p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v;
              __nv_bfloat162* vb = (__nv_bfloat162*)&v;
#pragma unroll
              for (int e = 0; e < 4; ++e)
                vb[e] = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * e]) * alpha, __uint_as_float(r[j + 2 * e + 1]) * alpha);
              *(uint4*)(crow + j) = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) crow[j] = __float2bfloat16(__uint_as_float(r[j]) * alpha);
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

extern "C" int hippo_nvfp4_tile_scales(const void* sf, void* out, long long rows, long long K, void* stream) {
  if (K % 64) return -1;
  long long rp = (rows + 127) / 128 * 128;
  long long total = rp * (K / 16);
  nvfp4_tile_scales_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)sf, (uint8_t*)out, rows, (int)(K / 16), rp);
  return (int)cudaGetLastError();
}

// A: [M, K/2] packed fp4 bytes, B: [N, K/2]; sfa/sfb: tiled scales (hippo_nvfp4_tile_scales); gsa/gsb: device fp32[1].
extern "C" int hippo_gemm_nvfp4(const void* A, const void* B, const void* sfa, const void* sfb, const float* gsa,
                                const float* gsb, void* C, int M, int N, int K, long long ldc, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 256 || (N % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)C & 15) || (ldc % 8)) return -2;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, A, (uint64_t)K / 2, (uint64_t)M, (uint64_t)K / 2, F_BKB, F_BM, 1, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, (uint64_t)K / 2, (uint64_t)N, (uint64_t)K / 2, F_BKB, F_BN, 1, true);
  if (rc) return rc;
  Fp4Params p;
  p.M = M; p.N = N; p.K = K; p.sfa = (const uint8_t*)sfa; p.sfb = (const uint8_t*)sfb; p.gsa = gsa; p.gsb = gsb;
  p.C = (__nv_bfloat16*)C; p.ldc = ldc;
  p.tiles_m = (M + F_BM - 1) / F_BM; p.tiles_n = (N + F_BN - 1) / F_BN;
  int tiles = p.tiles_m * p.tiles_n, sms = sm_count();
  int grid = tiles < sms ? tiles : sms;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  gemm_nvfp4_kernel<<<grid, F_THREADS, F_SMEM, (cudaStream_t)stream>>>(tmA, tmB, p);
  return (int)cudaGetLastError();
}
