// CTA-pair NVFP4 GEMM:  C[M,N] (+)= (A_fp4 * sfA) (B_fp4 * sfB)^T * gsA * gsB  on a 256 x 256 tile shared by two CTAs.
//
//   tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X, MMA shape 256 x 256 x 64
//
// A 128x128x64 FP4 MMA of the one-CTA kernel (gemm_fp4.cu) reads 8 KB of operands from shared memory in 64 tensor-pipe
// cycles, 128 bytes per clock, which is all the shared-memory bandwidth an SM has: that kernel stops at 2.1 PFLOP/s.
// Here each CTA of the pair stages its own 128 rows of A and only HALF of the 256 B rows (plus the scale tiles of its A
// rows and of all 256 B rows): per SM 8 KB of operand reads per 128x256x64 MMA, i.e. half the bytes per flop, and
// 38 KB instead of 72 KB of L2 -> shared-memory traffic per 128x256x256 slab.
//
// TMEM holds 512 columns: a 128 x 256 fp32 accumulator takes 256, the scale factors of the stages in flight take
// the rest (4 columns per 128-row tile and MMA: 16 for A, 32 for B per stage), so there is ONE accumulator. The
// epilogue therefore drains it into registers first (a thread holds its row as 128 packed bf16 pairs), hands TMEM back
// to the MMA issuer, and only then writes (or adds into) global memory while the next tile's MMAs run. No shared
// memory goes to the epilogue: five 38 KB stages.
//
// One thread cannot issue a slab's 12 scale copies (tcgen05.cp, shared memory -> TMEM), 4 MMAs and 2 commits as fast as
// the tensor pipe retires the MMAs: with all of them in the MMA thread the kernel ran at 2.9 PFLOP/s with the pipe idle
// two thirds of the time, without the copies (wrong results, timing only) at 4.8. So the copies have their own three
// warps (A tiles, lower and upper B tiles), each committing to a per-stage barrier the MMA thread waits on: 4.2 PFLOP/s.
//
// Per CTA (288 threads): warp 0 = TMA producer (all five loads of a stage are tiled TMA loads of local memory whose
// completion bytes land on the LEADER's barrier; the scale arrays are addressed as [tile * K/64 + k][128 x u32]
// tensors), warp 1 = MMA issuer (leader only) and TMEM owner, warps 2..5 = epilogue of the CTA's own 128 rows, warps
// 6..8 = scale copies (leader only; tcgen05.cp.cta_group::2 copies from both CTAs' shared memory into both CTAs'
// TMEM). Stage release and accumulator hand-over as in the bf16 pair kernel: two plain commits (own barrier, peer
// barrier), remote mbarrier arrives; no cluster-multicast qualifier. Every wait is bounded. Replaces the reference's
// Marlin W4A16 path like the one-CTA kernel.
#include "sm100.cuh"
#include "host_utils.h"
#include "cta_pair.cuh"
#include <cuda_bf16.h>
#include <stdlib.h>

namespace hippo {
namespace f2 {

constexpr int BM = 128;                 // rows per CTA; the pair covers 256
constexpr int BN = 256, BNH = 128;      // columns of the pair tile / B rows staged by each CTA
constexpr int BKB = 128;                // K slab: 128 bytes = 256 fp4 elements = 4 MMAs
constexpr int A_BYTES = BM * BKB, B_BYTES = BNH * BKB, SFA_BYTES = 4 * 512, SFB_BYTES = 2 * 4 * 512;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;          // 38 KB
constexpr int THREADS = 288;            // TMA, MMA, 4 epilogue warps, 3 scale-copy warps
constexpr int COPY_WARP0 = 6, COPY_WARPS = 3;
constexpr int TMEM_SF0 = 256;           // the accumulator uses columns [0, 256); 48 scale columns per stage follow
// Fused collective modes (same protocol as the one-CTA kernel of gemm_fp4.cu, whose launchers route here):
//   P_COMM_AG  A is this rank's gathered FP4 buffer, filled shard by shard by every rank's quantise-and-push kernel; the
//              producer acquires (bounded) the arrival counter of its 128-row block before the block's first load and
//              the epilogue applies the source rank's tensor scale.
//   P_COMM_RS  partial tiles go to the staging slot [this rank] of the rank that owns the rows: the epilogue lays each
//              warp's 32 x 256 slab out in shared memory (4 stages instead of 5 make room) and every lane sends its row
//              with one bulk async copy; one completion wait + counter release per owner shard; after its last tile
//              every CTA joins the reduction of the local rows.
constexpr int P_COMM_NONE = 0, P_COMM_AG = 1, P_COMM_RS = 2;
constexpr int RS_PITCH = 528, RS_SLABS = 4 * 32 * RS_PITCH;   // slab rows 512 bytes at a bank-conflict-free pitch
template <int COMM> __host__ __device__ constexpr int stages_of() { return COMM == P_COMM_RS ? 4 : 5; }
template <int COMM> __host__ __device__ constexpr int smem_of() {
  return stages_of<COMM>() * STAGE_BYTES + (COMM == P_COMM_RS ? RS_SLABS : 0) + 1024 + 256;
}
static_assert(STAGE_BYTES % 1024 == 0, "operand tiles must stay 1024-byte aligned (128-byte swizzle)");
static_assert(TMEM_SF0 + 5 * 48 <= 512, "scale-factor columns must fit behind the accumulator");
static_assert(smem_of<P_COMM_NONE>() <= 227 * 1024 && smem_of<P_COMM_RS>() <= 227 * 1024, "shared memory of one CTA");

struct PairParams {
  int M, N, K;                          // K in elements (multiple of 256)
  const float* gsa; const float* gsb;
  __nv_bfloat16* C; long long ldc;
  int accumulate;                       // C += result (weight-gradient products)
  int tiles_m, tiles_n;                 // pair tiles
  // fused collectives
  int world, rank, rows_per_shard;      // rows_per_shard: a multiple of 256
  const uint32_t* flags; uint32_t target; long long wait_cycles;          // AG: flags[128-row block of the gathered A]
  void* stage_peer[8]; uint32_t* rs_flag_peer[8]; uint32_t rs_target; void* out_local;   // RS
};

__device__ __forceinline__ uint32_t p_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// bounded spin on a monotonic counter written by other GPUs
__device__ __forceinline__ bool p_wait_counter(const uint32_t* p, uint32_t target, long long limit, int detail) {
  if ((int32_t)(p_ld_acquire_sys(p) - target) >= 0) return true;
  long long t0 = clock64();
  while ((int32_t)(p_ld_acquire_sys(p) - target) < 0) {
    if (clock64() - t0 > limit) { report(kWaitPeerFlag, detail); return false; }
    __nanosleep(64);
  }
  return true;
}

__device__ __forceinline__ void mma_nvf4_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
      : "memory");
}
// shared memory -> TMEM copy of one 512-byte scale tile in BOTH CTAs of the pair (each from its own shared memory at
// the same offset into its own TMEM), replicated to the four 32-lane groups
__device__ __forceinline__ void tc_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

template <int COMM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_nvfp4_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                      const __grid_constant__ PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int STAGES = stages_of<COMM>();
  uint8_t* epi_stage = smem + STAGES * STAGE_BYTES;            // P_COMM_RS only: 4 warps x [32 rows][RS_PITCH]
  uint64_t* full = (uint64_t*)(epi_stage + (COMM == P_COMM_RS ? RS_SLABS : 0));   // used in the leader only
  uint64_t* empty = full + STAGES;                             // one set per CTA
  uint64_t* tfull = empty + STAGES;                            // one per CTA
  uint64_t* tempty = tfull + 1;                                // used in the leader only (8 arrivals)
  uint64_t* sf_full = tempty + 1;                              // leader only: scale tiles of a stage are in TMEM
  uint32_t* tmem_slot = (uint32_t*)(sf_full + STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = p.K / 256;
  const int k64 = p.K / 64;
  const int cid = (int)blockIdx.x >> 1, n_clusters = (int)gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&sf_full[s], COPY_WARPS); }
    mbar_init(tfull, 1); mbar_init(tempty, 8);
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB); prefetch_tmap(&tmSFA); prefetch_tmap(&tmSFB);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                     // both CTAs' barriers are initialised before any remote arrive
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int GROUP = 8;                  // 8 pair tiles (2048 rows) share each column sweep
    int tiles_m = p.tiles_m, base_m = 0;
    if (COMM != P_COMM_NONE) {            // shard by shard: AG in arrival order (own, rank-1, ...), RS remote owners first
      const int tms = p.rows_per_shard / (2 * BM);
      const int per_shard = tms * p.tiles_n;
      const int si = t / per_shard;
      t -= si * per_shard;
      const int shard = (COMM == P_COMM_AG) ? (p.rank - si + p.world) % p.world : (p.rank + 1 + si) % p.world;
      base_m = shard * tms; tiles_m = tms;
    }
    int per_group = GROUP * p.tiles_n;
    int g = t / per_group, r = t % per_group;
    int gm = min(GROUP, tiles_m - g * GROUP);
    tm = base_m + g * GROUP + r % gm;
    tn = r / gm;
  };

  // One K slab has 12 scale tiles (4 MMAs x (1 tile of A rows + 2 tiles of B rows)); copy warp `part` moves 4 of them,
  // shared memory -> TMEM of both CTAs: part 0 the A tiles, parts 1 and 2 the tiles of B rows 0..127 and 128..255.
  auto issue_scale_copies = [&](int j, int part) {
    const int s = j % STAGES;
    const uint32_t src = smem_u32(smem + s * STAGE_BYTES) + A_BYTES + B_BYTES + part * SFA_BYTES;
    const uint32_t t_sf = tmem_base + TMEM_SF0 + s * 48;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t dst = part == 0 ? t_sf + k * 4 : t_sf + 16 + k * 8 + (part - 1) * 4;
      // a scale tile is 32 rows x 16 bytes, rows contiguous: 8-row groups 128 bytes apart, no swizzle
      tc_cp_32x128b_warpx4_pair(dst, make_smem_desc_noswizzle(src + k * 512, 16, 128));
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      int it = 0, last_rb = -1;
      bool ok = true;
      for (int t = cid; t < num_tiles && ok; t += n_clusters) {
        int tm, tn; tile_coord(t, tm, tn);
        const int rb = tm * 2 + (int)rank;                     // this CTA's 128-row block of A
        const int cb = tn * 2 + (int)rank;                     // this CTA's 128-row block of B
        if (COMM == P_COMM_AG && rb != last_rb) {              // one acquire per new row block of a remote shard
          const int bps = p.rows_per_shard / BM;
          if (rb / bps != p.rank) {                            // own rows were written by the previous local kernel
            ok = p_wait_counter(p.flags + rb, p.target, p.wait_cycles, rb);
            asm volatile("fence.proxy.async;" ::: "memory");   // remote generic-proxy writes -> TMA reads
            if (!ok) break;
          }
          last_rb = rb;
        }
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          int s = it % STAGES; uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&empty[s], ph ^ 1, kWaitSmemEmpty, it);
          if (!ok) break;
          if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          uint8_t* sa = smem + s * STAGE_BYTES; uint8_t* sb = sa + A_BYTES;
          uint8_t* ssa = sb + B_BYTES; uint8_t* ssb = ssa + SFA_BYTES;
          tma_load_2d_pair(sa, &tmA, bar, kb * BKB, rb * BM);
          tma_load_2d_pair(sb, &tmB, bar, kb * BKB, cb * BNH);
          tma_load_2d_pair(ssa, &tmSFA, bar, 0, rb * k64 + kb * 4);
          tma_load_2d_pair(ssb, &tmSFB, bar, 0, (tn * 2) * k64 + kb * 4);              // scales of B rows 0..127
          tma_load_2d_pair(ssb + 4 * 512, &tmSFB, bar, 0, (tn * 2 + 1) * k64 + kb * 4);  // and of rows 128..255
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_nvf4(2 * BM, BN);
      int it = 0, tl = 0;
      bool ok = true;
      for (int t = cid; t < num_tiles && ok; t += n_clusters, ++tl) {
        ok = mbar_wait(tempty, (tl & 1) ^ 1, kWaitTmemEmpty, tl);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          int s = it % STAGES; uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&sf_full[s], ph, kWaitTmaFull, it);      // operands landed and scales are in TMEM
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + A_BYTES;
          const uint32_t t_sfa = tmem_base + TMEM_SF0 + s * 48, t_sfb = t_sfa + 16;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint64_t ad = make_smem_desc(sa + k * 32, 16, 1024);
            uint64_t bd = make_smem_desc(sb + k * 32, 16, 1024);
            mma_nvf4_ss_pair(tmem_base, ad, bd, idesc, t_sfa + k * 4, t_sfb + k * 8, (kb | k) ? 1u : 0u);
          }
          const uint32_t e = smem_u32(&empty[s]);
          tc_commit_pair(e);                                    // stage free in this CTA ...
          tc_commit_pair(map_to_cta(e, 1));                     // ... and in the peer
        }
        if (ok) {
          const uint32_t f = smem_u32(tfull);
          tc_commit_pair(f);
          tc_commit_pair(map_to_cta(f, 1));
        }
      }
    }
  } else if (warp >= COPY_WARP0) {
    if (lane == 0 && leader) {
      const int part = warp - COPY_WARP0;
      const int total_its = cid < num_tiles ? ((num_tiles - cid + n_clusters - 1) / n_clusters) * kblocks : 0;
      for (int it = 0; it < total_its; ++it) {
        const int s = it % STAGES; const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&full[s], ph, kWaitTmaFull, it)) break;
        tc_fence_after();
        issue_scale_copies(it, part);
        tc_commit_pair(smem_u32(&sf_full[s]));
      }
    }
  } else {
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const float gsb = *p.gsb;
    float alpha = (COMM == P_COMM_AG) ? 0.f : (*p.gsa) * gsb;
    int tl = 0;
    int rs_pending = 0;                     // P_COMM_RS: arrivals of the current owner shard stored but not yet released
    bool ok = true;
    for (int t = cid; t < num_tiles && ok; t += n_clusters, ++tl) {
      int tm, tn; tile_coord(t, tm, tn);
      ok = mbar_wait(tfull, tl & 1, kWaitTmemFull, tl);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
      if (COMM == P_COMM_AG) {              // the tensor scale of the source shard was pushed before its counters were released
        float g;
        asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(g) : "l"(p.gsa + (tm * 2 * BM) / p.rows_per_shard) : "memory");
        alpha = g * gsb;
      }
      if (COMM == P_COMM_RS) {
        uint8_t* slab = epi_stage + (warp - 2) * 32 * RS_PITCH;
        tma_store_wait_read<0>();                                          // the previous tile's rows have left the slab
        __syncwarp();
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
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
            *(uint4*)(slab + lane * RS_PITCH + (c + j) * 2) = v;
          }
        }
        fence_proxy_async();                                               // generic-proxy slab writes -> bulk copy reads
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(tempty), 0));   // accumulator back to the leader
        const int row_base = (tm * 2 + (int)rank) * BM + q * 32;
        const int owner = row_base / p.rows_per_shard;
        const int ncols = min(BN, p.N - tn * BN);                          // multiple of 8
        if (row_base + lane < p.M) {
          __nv_bfloat16* dst = (__nv_bfloat16*)p.stage_peer[owner] +
                               ((long long)p.rank * p.rows_per_shard + (row_base + lane - owner * p.rows_per_shard)) * p.N + tn * BN;
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                       ::"l"(dst), "r"(smem_u32(slab + lane * RS_PITCH)), "r"((uint32_t)(ncols * 2)) : "memory");
        }
        tma_store_commit();
        // The counters follow the one-CTA kernel's convention (one arrival per warp and 128-column tile), so the host's
        // cumulative targets do not depend on which kernel ran: a pair tile counts for the 128-column tiles it covers.
        rs_pending += ncols > 128 ? 2 : 1;
        const int tnext = t + n_clusters;
        int owner_next = -1;
        if (tnext < num_tiles) {
          int tm2, tn2; tile_coord(tnext, tm2, tn2);
          owner_next = ((tm2 * 2 + (int)rank) * BM + q * 32) / p.rows_per_shard;
        }
        if (owner_next != owner) {                                         // one completion wait + release per owner shard
          tma_store_wait<0>();
          __threadfence_system();
          __syncwarp();
          if (lane == 0)
            asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.rs_flag_peer[owner] + p.rank), "r"((uint32_t)rs_pending) : "memory");
          rs_pending = 0;
        }
      } else {
        uint32_t pk[BN / 2];                                               // this thread's row, packed bf16 pairs
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * j]) * alpha, __uint_as_float(r[2 * j + 1]) * alpha);
            pk[c * 16 + j] = *(const uint32_t*)&h;
          }
        }
        // the accumulator is in registers now: hand TMEM back to the leader before touching global memory
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(tempty), 0));
        const int row = (tm * 2 + (int)rank) * BM + q * 32 + lane;
        if (row < p.M) {
          __nv_bfloat16* crow = p.C + (long long)row * p.ldc + tn * BN;
          const int ncols = min(BN, p.N - tn * BN);                        // multiple of 8
#pragma unroll
          for (int c = 0; c < BN / 8; ++c) {                               // 16-byte pieces of the row
            if (c * 8 < ncols) {
              uint4 v = make_uint4(pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]);
              if (p.accumulate) {
                const uint4 old = *(const uint4*)(crow + c * 8);
                __nv_bfloat162* vb = (__nv_bfloat162*)&v;
                const __nv_bfloat162* ob = (const __nv_bfloat162*)&old;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 x = __bfloat1622float2(vb[e]), o = __bfloat1622float2(ob[e]);
                  vb[e] = __floats2bfloat162_rn(x.x + o.x, x.y + o.y);
                }
              }
              *(uint4*)(crow + c * 8) = v;
            }
          }
        }
      }
    }
  }
  // Neither CTA may leave (or free its TMEM) while the other can still read its shared memory or signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
  if (COMM == P_COMM_RS) {
    // reduction of the rows this rank owns: wait (bounded) for every source, then sum the staging slots
    if ((int)threadIdx.x < p.world)
      p_wait_counter(p.rs_flag_peer[p.rank] + threadIdx.x, p.rs_target, p.wait_cycles, 100 + threadIdx.x);
    __syncthreads();
    const long long nvec = (long long)p.rows_per_shard * p.N / 8;
    const uint4* stage = (const uint4*)p.stage_peer[p.rank];
    uint4* out = (uint4*)p.out_local;
    const long long stride = (long long)gridDim.x * THREADS;
    for (long long v0 = (long long)blockIdx.x * THREADS + threadIdx.x; v0 < nvec; v0 += stride * 4) {
      float acc[4][8];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
      for (int sidx = 0; sidx < p.world; ++sidx) {
        uint4 x[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {                                      // 4 independent loads in flight per source
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

template <int COMM>
static int launch_pair(const void* A, const void* B, const void* sfa, const void* sfb, PairParams p, cudaStream_t stream) {
  const int k64 = p.K / 64;
  CUtensorMap tmA, tmB, tmSFA, tmSFB;
  int rc = make_tmap_2d(&tmA, A, (uint64_t)p.K / 2, (uint64_t)p.M, (uint64_t)p.K / 2, BKB, BM, 1, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, B, (uint64_t)p.K / 2, (uint64_t)p.N, (uint64_t)p.K / 2, BKB, BNH, 1, true);
  if (rc) return rc;
  // scale arrays as [tile * K/64 + k][128 x 4-byte words]; one load = the four k-groups of a K slab (2 KB, contiguous)
  rc = make_tmap_2d(&tmSFA, sfa, 128, (uint64_t)((p.M + 127) / 128) * k64, 512, 128, 4, 4, false);
  if (rc) return rc;
  rc = make_tmap_2d(&tmSFB, sfb, 128, (uint64_t)((p.N + 127) / 128) * k64, 512, 128, 4, 4, false);
  if (rc) return rc;
  p.tiles_m = (p.M + 2 * BM - 1) / (2 * BM); p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  int clusters = sm_count() / 2;
  if (clusters < 1) clusters = 1;
  if (tiles < clusters) clusters = tiles;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_2sm_kernel<COMM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_of<COMM>());
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  gemm_nvfp4_2sm_kernel<COMM><<<2 * clusters, THREADS, smem_of<COMM>(), stream>>>(tmA, tmB, tmSFA, tmSFB, p);
  return (int)cudaGetLastError();
}

}  // namespace f2
}  // namespace hippo

using namespace hippo;

// A: [M, K/2] packed fp4 bytes, B: [N, K/2]; sfa / sfb: scale tiles [ceil(rows/128)][K/64][512]; gsa / gsb: device
// fp32[1]; C: bf16 [M, ldc]. accumulate != 0 adds into C. Returns -3 for shapes the pair kernel does not take
// (fewer than 256 rows or columns): the caller falls back to the one-CTA kernel.
extern "C" int hippo_gemm_nvfp4_pair(const void* A, const void* B, const void* sfa, const void* sfb, const float* gsa,
                                     const float* gsb, void* C, int M, int N, int K, long long ldc, int accumulate,
                                     void* stream) {
  using namespace f2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 256 || (N % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)C & 15) || (ldc % 8) ||
      ((uintptr_t)sfa & 15) || ((uintptr_t)sfb & 15)) return -2;
  if (M < 2 * BM || N < BN) return -3;
  PairParams p = {};
  p.M = M; p.N = N; p.K = K; p.gsa = gsa; p.gsb = gsb; p.C = (__nv_bfloat16*)C; p.ldc = ldc; p.accumulate = accumulate;
  return launch_pair<P_COMM_NONE>(A, B, sfa, sfb, p, (cudaStream_t)stream);
}

// All-gather -> GEMM on the pair kernel; arguments as hippo_allgather_gemm_nvfp4 (gemm_fp4.cu), which routes here when
// rows_per_shard is a multiple of 256 and N >= 256.
extern "C" int hippo_allgather_gemm_nvfp4_pair(const void* gathered, const void* flags, int world, int rank,
                                               int rows_per_shard, const void* B, const void* sfb, const float* gsb,
                                               void* C, long long ldc, int N, int K, unsigned target,
                                               long long wait_cycles, void* stream) {
  using namespace f2;
  if (world < 1 || world > 8 || rows_per_shard % (2 * BM) || K % 512 || (N % 8) || (ldc % 8) || N < BN) return -2;
  const int M = world * rows_per_shard;
  const uint8_t* base = (const uint8_t*)gathered;
  const long long sf_off = (long long)M * (K / 2), gs_off = sf_off + (long long)M * (K / 16);
  PairParams p = {};
  p.M = M; p.N = N; p.K = K; p.gsa = (const float*)(base + gs_off); p.gsb = gsb; p.C = (__nv_bfloat16*)C; p.ldc = ldc;
  p.world = world; p.rank = rank; p.rows_per_shard = rows_per_shard;
  p.flags = (const uint32_t*)flags; p.target = target; p.wait_cycles = wait_cycles > 0 ? wait_cycles : kWaitCycles;
  return launch_pair<P_COMM_AG>(base, B, base + sf_off, sfb, p, (cudaStream_t)stream);
}

// GEMM -> reduce-scatter on the pair kernel; arguments as hippo_gemm_reduce_scatter_nvfp4 (gemm_fp4.cu).
extern "C" int hippo_gemm_reduce_scatter_nvfp4_pair(const void* A, const void* sfa, const float* gsa, const void* B,
                                                    const void* sfb, const float* gsb, void* const* stage_ptrs,
                                                    void* const* flag_ptrs, int world, int rank, int rows_per_shard,
                                                    void* out_local, int N, int K, unsigned target,
                                                    long long wait_cycles, void* stream) {
  using namespace f2;
  if (world < 1 || world > 8 || rows_per_shard % (2 * BM) || K % 256 || (N % 8) || N < BN) return -2;
  PairParams p = {};
  p.M = world * rows_per_shard; p.N = N; p.K = K; p.gsa = gsa; p.gsb = gsb; p.C = nullptr; p.ldc = N;
  p.world = world; p.rank = rank; p.rows_per_shard = rows_per_shard;
  p.wait_cycles = wait_cycles > 0 ? wait_cycles : kWaitCycles;
  for (int r = 0; r < world; ++r) { p.stage_peer[r] = stage_ptrs[r]; p.rs_flag_peer[r] = (uint32_t*)flag_ptrs[r]; }
  p.rs_target = target; p.out_local = out_local;
  return launch_pair<P_COMM_RS>(A, B, sfa, sfb, p, (cudaStream_t)stream);
}
