// CTA-pair bf16 GEMM on tcgen05 tensor cores (sm_100a): two CTAs on neighbouring SMs share one 256x256 tile.
//
// A 128x256 one-CTA tile reads 12 KB of operands from shared memory per 128x256x16 MMA, which caps the
// tensor pipe at the shared-memory bandwidth (~0.8 of peak). With `cta_group::2` each CTA of the pair stages
// its own 128 rows of A and only HALF of the B tile (128 of the 256 columns); the MMA issued by the leader
// CTA (cluster rank 0) runs on both SMs, every SM reading 8 KB per step, and the accumulator of the pair is
// split by rows: rows 0..127 in the leader's TMEM, rows 128..255 in the peer's.
//
// Per CTA (192 threads): warp 0 = TMA producer (own A rows, own B half; the completion bytes of both CTAs land
// on the LEADER's full barrier), warp 1 = MMA issuer (leader only) and TMEM owner, warps 2..5 = epilogue of the
// CTA's own 128 rows. The leader's MMA thread releases shared-memory stages and publishes accumulators by
// committing to the barrier of each CTA in turn (two plain commits, no cluster-multicast qualifier anywhere);
// the peer's epilogue warps hand the accumulator back with a remote mbarrier arrive. 6 stages of 32 KB, two
// 256-column accumulators. All loads are plain TMA loads of local memory. Every wait is bounded.
// Replaces the reference's cuBLAS calls behind F.linear / torch.mm (qkv_proj, o_proj, FFN, LCE, Newton-Schulz).
#include "sm100.cuh"
#include "host_utils.h"
#include "gemm_params.h"
#include "gemm_comm.cuh"
#include "cta_pair.cuh"
#include <stdlib.h>

namespace hippo {
namespace sm2 {

constexpr int BM = 128;            // rows per CTA; the pair covers 256
constexpr int BN = 256;            // columns of the pair tile
constexpr int BNH = BN / 2;        // columns of B staged by each CTA
constexpr int BK = 64, UMMA_K = 16, STAGES = 6;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
// COMM_RS: 4 pipeline stages + the epilogue slabs (4 warps x 32 rows of 512 bytes at a 528-byte pitch: 16-byte stores of a
// quarter warp then fall on distinct banks, and every row stays a 16-byte aligned source of a bulk copy)
constexpr int RS_PITCH = 528, RS_SLABS = 4 * 32 * RS_PITCH;
constexpr int SMEM_RS = 4 * STAGE_BYTES + RS_SLABS + 1024 + 256;

__device__ __forceinline__ void mma_f16_ss_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// COMM == COMM_RS: GEMM -> reduce-scatter in this kernel. Pair tiles are walked remote owners first (rank+1, ...), own
// rows last; the epilogue of every CTA lays its warps' 32 x 256 slabs out in shared memory (the space of pipeline stages
// 4 and 5; the main loop runs on 4 stages) and writes 512-byte rows into the staging slot [this rank] of the rank that
// owns the rows, then releases that rank's per-source counter; after its last tile every CTA joins the reduction of the
// local rows (bounded wait for all sources, sum of the slots).
// COMM == COMM_AG: all-gather -> GEMM in this kernel. The first cp.comm_ctas CTAs (whole clusters) run the bulk-copy
// role of gemm_comm.cuh instead of computing; the GEMM clusters walk the 256-row pair tiles shard by shard in arrival
// order, every CTA's TMA producer acquiring (bounded) the arrival counter of ITS 128-row block before the block's first
// load; tiles of the own shard read x_local in place through tmOwn. All loads are plain TMA loads of local memory.
// COMM == EPI_LCE: no collective. The logits GEMM of the linear + cross-entropy head: the epilogue rounds every accumulator
// row to bf16 (the stored logits), and, while the 256 values of the row are in registers, folds them into the row's
// running (max, sum exp) of this tile and picks the logit at the row's target column; the per-tile pairs go to
// p.lce_part[tile column][row] and are merged per row by ce_part_merge_kernel (lce_fused.cu). The fp32 logits never
// reach global memory and no separate pass over them computes the statistics.
template <bool A_KMAJOR, bool B_KMAJOR, int COMM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_bf16_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p,
                     const __grid_constant__ CommParams cp, const __grid_constant__ CUtensorMap tmOwn) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + (COMM == COMM_RS ? 4 * STAGE_BYTES + RS_SLABS : STAGES * STAGE_BYTES));   // used in the leader only
  uint64_t* empty = full + STAGES;                             // one per CTA
  uint64_t* tfull = empty + STAGES;                            // one per CTA
  uint64_t* tempty = tfull + 2;                                // used in the leader only (8 arrivals)
  uint32_t* tmem_slot = (uint32_t*)(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  // pair tiles (256 x 256); a symmetric-output launch enumerates only the tiles on or below the diagonal
  const int out_tiles = p.sym_lower ? p.tiles_m * (p.tiles_m + 1) / 2 : p.tiles_m * p.tiles_n;
  const int kblocks_all = (p.K + BK - 1) / BK;
  // split-K: work item t = slice * out_tiles + tile; every slice covers kb_per k-blocks (the last one what is left)
  const int ksplit = p.ksplit > 1 ? p.ksplit : 1;
  const int kb_per = (kblocks_all + ksplit - 1) / ksplit;
  const int num_tiles = out_tiles * ksplit;
  constexpr int NST = (COMM == COMM_RS) ? 4 : STAGES;              // RS: stages 4 and 5 are the epilogue staging area
  uint8_t* epi_stage = smem + 4 * STAGE_BYTES;                      // COMM_RS only: 4 warps x [32][512 B]
  const int comm_clusters = (COMM == COMM_AG) ? cp.comm_ctas >> 1 : 0;
  const int cid = ((int)blockIdx.x >> 1) - comm_clusters, n_clusters = ((int)gridDim.x >> 1) - comm_clusters;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 8); }
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB);
    if (COMM == COMM_AG) prefetch_tmap(&tmOwn);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                     // both CTAs' barriers are initialised before any remote arrive
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;  // whole TMEM of the SM: the same address in both CTAs

  auto tile_coord = [&](int t, int& tm, int& tn) {
    if (p.sym_lower) {                    // row-major walk of the lower triangle: t = tm (tm + 1) / 2 + tn
      tm = (int)((sqrtf(8.f * (float)t + 1.f) - 1.f) * 0.5f);
      while ((tm + 1) * (tm + 2) / 2 <= t) ++tm;
      while (tm * (tm + 1) / 2 > t) --tm;
      tn = t - tm * (tm + 1) / 2;
      return;
    }
    const int GROUP = 8;                  // 8 pair-tiles (2048 rows) share each column sweep
    int tiles_m = p.tiles_m, base_m = 0;
    if (COMM == COMM_AG || COMM == COMM_RS) {   // shard by shard: AG in arrival order (own, rank-1, ...), RS remote owners first
      const int tms = cp.rows_per_shard / (2 * BM);
      const int per_shard = tms * p.tiles_n;
      const int si = t / per_shard;
      t -= si * per_shard;
      const int shard = (COMM == COMM_AG) ? (cp.rank - si + cp.world) % cp.world : (cp.rank + 1 + si) % cp.world;
      base_m = shard * tms; tiles_m = tms;
    }
    int per_group = GROUP * p.tiles_n;
    int g = t / per_group, r = t % per_group;
    int gm = min(GROUP, tiles_m - g * GROUP);
    tm = base_m + g * GROUP + r % gm;
    tn = r / gm;
  };

  if (COMM == COMM_AG && (int)blockIdx.x < cp.comm_ctas) {
    if (threadIdx.x == 0) ag_copy_role<STAGE_BYTES, BM, STAGES>(smem, full, cp, p.K, (int)blockIdx.x);
  } else
  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      int last_rb = -1;
      for (int t = cid; t < num_tiles && ok; t += n_clusters) {
        int tm, tn; tile_coord(t % out_tiles, tm, tn);
        const int row0 = (tm * 2 + (int)rank) * BM;            // this CTA's rows of A / C
        const int col0 = tn * BN + (int)rank * BNH;            // this CTA's half of the B tile
        const int kb0 = (t / out_tiles) * kb_per, kb1 = min(kblocks_all, kb0 + kb_per);
        bool own_tile = false;
        if (COMM == COMM_AG) {
          const int rb = tm * 2 + (int)rank;                   // this CTA's 128-row block of the gathered A
          const int own_lo = cp.rank * (cp.rows_per_shard / BM);
          own_tile = rb >= own_lo && rb < own_lo + cp.rows_per_shard / BM;
          if (!own_tile && rb != last_rb) {                    // one acquire per new row block
            ok = wait_counter(cp.flag_peer[cp.rank] + rb, cp.target, cp.wait_cycles, rb);
            asm volatile("fence.proxy.async;" ::: "memory");   // remote async-proxy writes -> TMA reads
            last_rb = rb;
            if (!ok) break;
          }
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          int s = it % NST; uint32_t ph = (it / NST) & 1;
          ok = mbar_wait(&empty[s], ph ^ 1, kWaitSmemEmpty, it);
          if (!ok) break;
          if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          uint8_t* sa = smem + s * STAGE_BYTES; uint8_t* sb = sa + A_BYTES;
          if (COMM == COMM_AG && own_tile) {
            tma_load_2d_pair(sa, &tmOwn, bar, kb * BK, row0 - cp.rank * cp.rows_per_shard);
          } else if (A_KMAJOR) {
            tma_load_2d_pair(sa, &tmA, bar, kb * BK, row0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tmA, bar, row0 + j * 64, kb * BK);
          }
          if (B_KMAJOR) {
            tma_load_2d_pair(sb, &tmB, bar, kb * BK, col0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tmB, bar, col0 + j * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_f16(2 * BM, BN, 1, A_KMAJOR ? 0 : 1, B_KMAJOR ? 0 : 1);
      int it = 0, tl = 0;
      bool ok = true;
      for (int t = cid; t < num_tiles && ok; t += n_clusters) {
        const int tl_now = tl++;
        int acc = tl_now & 1; uint32_t aph = (tl_now >> 1) & 1;
        ok = mbar_wait(&tempty[acc], aph ^ 1, kWaitTmemEmpty, tl_now);
        if (!ok) break;
        tc_fence_after();
        uint32_t d_tmem = tmem_base + acc * BN;
        const int kb0 = (t / out_tiles) * kb_per, kb1 = min(kblocks_all, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          int s = it % NST; uint32_t ph = (it / NST) & 1;
          ok = mbar_wait(&full[s], ph, kWaitTmaFull, it);
          if (!ok) break;
          tc_fence_after();
          uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t ad = A_KMAJOR ? make_smem_desc(sa + k * 32, 16, 1024) : make_smem_desc(sa + k * 2048, 8192, 1024);
            uint64_t bd = B_KMAJOR ? make_smem_desc(sb + k * 32, 16, 1024) : make_smem_desc(sb + k * 2048, 8192, 1024);
            mma_f16_ss_pair(d_tmem, ad, bd, idesc, ((kb - kb0) | k) ? 1u : 0u);
          }
          const uint32_t e = smem_u32(&empty[s]);
          tc_commit_pair(e);                                    // stage free in this CTA ...
          tc_commit_pair(map_to_cta(e, 1));                     // ... and in the peer
        }
        if (ok) {
          const uint32_t f = smem_u32(&tfull[acc]);
          tc_commit_pair(f);
          tc_commit_pair(map_to_cta(f, 1));
        }
      }
    }
  } else {
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    int tl = 0;
    int rs_pending = 0;                     // COMM_RS: tiles of the current owner shard stored but not yet released
    bool ok = true;
    for (int t = cid; t < num_tiles && ok; t += n_clusters) {
      int tm, tn; tile_coord(t % out_tiles, tm, tn);
      GemmParams pe = p;                                          // split-K: this slice's partial-product plane
      if (ksplit > 1) pe.C = (float*)p.C + (long long)(t / out_tiles) * p.M * p.ldc;
      const int tl_now = tl++;
      int acc = tl_now & 1; uint32_t aph = (tl_now >> 1) & 1;
      ok = mbar_wait(&tfull[acc], aph, kWaitTmemFull, tl_now);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = (tm * 2 + (int)rank) * BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      if (COMM == COMM_RS) {
        // The warp lays its 32 x 256 slab out in shared memory, hands the accumulator back, and every lane sends its own
        // row (512 contiguous bytes) to the owner's staging slot with one bulk async copy: the remote stores are in
        // flight while the warp drains the next tile instead of blocking it for an NVLink round trip per instruction.
        uint8_t* slab = epi_stage + (warp - 2) * 32 * RS_PITCH;
        tma_store_wait_read<0>();                                            // the previous tile's rows have left the slab
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
              vb[e] = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * e]) * p.alpha, __uint_as_float(r[j + 2 * e + 1]) * p.alpha);
            *(uint4*)(slab + lane * RS_PITCH + (c + j) * 2) = v;
          }
        }
        fence_proxy_async();                                                 // generic-proxy slab writes -> bulk copy reads
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));   // accumulator back to the leader
        const int row_base = (tm * 2 + (int)rank) * BM + q * 32;
        const int owner = row_base / cp.rows_per_shard;
        const int ncols = min(BN, p.N - tn * BN);                            // multiple of 8
        if (row_base + lane < p.M) {
          __nv_bfloat16* dst = (__nv_bfloat16*)cp.buf_peer[owner] +
                               ((long long)cp.rank * cp.rows_per_shard + (row_base + lane - owner * cp.rows_per_shard)) * p.N + tn * BN;
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                       ::"l"(dst), "r"(smem_u32(slab + lane * RS_PITCH)), "r"((uint32_t)(ncols * 2)) : "memory");
        }
        tma_store_commit();
        // One completion wait + counter release per OWNER SHARD, not per tile: the owner only starts its reduction when
        // all of a source's tiles have landed, so the remote-write round trip is paid once per shard.
        ++rs_pending;
        const int tnext = t + n_clusters;
        int owner_next = -1;
        if (tnext < num_tiles) {
          int tm2, tn2; tile_coord(tnext % out_tiles, tm2, tn2);
          owner_next = ((tm2 * 2 + (int)rank) * BM + q * 32) / cp.rows_per_shard;
        }
        if (owner_next != owner) {
          tma_store_wait<0>();                                               // this lane's rows have landed
          __threadfence_system();
          __syncwarp();
          if (lane == 0) red_release_sys_add(cp.flag_peer[owner] + cp.rank, (uint32_t)rs_pending);
          rs_pending = 0;
        }
        continue;
      }
      if (COMM == EPI_LCE) {
        // thread = row: online (max, sum exp) over the tile's columns of the bf16-rounded logits, target logit pick
        float mrow = -INFINITY, srow = 0.f, tzv = 0.f;
        const long long tg = row < p.M ? p.lce_target[row] : -1;
        const int tcol = (tg >= (long long)tn * BN && tg < (long long)(tn + 1) * BN) ? (int)(tg - (long long)tn * BN) : -1;
        pe.alpha = 1.f;                                                      // applied here, before the rounding
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          const int col0 = tn * BN + c;
          if (col0 >= p.N) break;                                            // uniform over the warp
          uint32_t r[32];
          EpiPrefetch pre;
          tmem_ld_32x32(taddr + c, r);
          tc_wait_ld();
          float cm = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float f = __bfloat162float(__float2bfloat16(__uint_as_float(r[j]) * p.alpha));
            r[j] = __float_as_uint(f);
            if (col0 + j < p.N) cm = fmaxf(cm, f);
            if (c + j == tcol) tzv = f;
          }
          if (cm > mrow) { srow *= __expf(mrow - cm); mrow = cm; }           // mrow = -inf: srow is 0 and stays 0
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) srow += __expf(__uint_as_float(r[j]) - mrow);
          epi_store(pe, r, row, col0, pre);                                  // exact: the values are bf16 already
        }
        if (row < p.M) {
          p.lce_part[(long long)tn * p.M + row] = make_float2(mrow, srow);
          if (tcol >= 0) p.lce_tz[row] = tzv;
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        EpiPrefetch pre;
        const int col0 = tn * BN + c;
        tmem_ld_32x32(taddr + c, r);
        epi_prefetch(pe, row, col0, pre);         // addends travel while the TMEM load completes
        tc_wait_ld();
        epi_store(pe, r, row, col0, pre);
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));   // hand the accumulator back to the leader
    }
  }
  // Neither CTA may leave (or free its TMEM) while the other can still read its shared memory or signal its barriers.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
  if (COMM == COMM_RS) {
    // ---- reduction of the rows this rank owns: wait for every source, then sum the staging slots
    if ((int)threadIdx.x < cp.world)
      wait_counter(cp.flag_peer[cp.rank] + threadIdx.x, cp.target, cp.wait_cycles, 100 + threadIdx.x);
    __syncthreads();
    const long long nvec = (long long)cp.rows_per_shard * p.N / 8;
    const uint4* stage = (const uint4*)cp.buf_peer[cp.rank];
    uint4* out = (uint4*)cp.out_local;
    const long long stride = (long long)gridDim.x * THREADS;
    for (long long v0 = (long long)blockIdx.x * THREADS + threadIdx.x; v0 < nvec; v0 += stride * 4) {
      float acc[4][8];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
      for (int sidx = 0; sidx < cp.world; ++sidx) {
        uint4 x[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {                        // 4 independent loads in flight per source
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

template <bool AK, bool BK_, int COMM>
static int launch(const void* A, const void* B, long long lda, long long ldb, GemmParams p, int max_ctas,
                  const CommParams& cp, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc;
  if (AK) rc = make_tmap_2d(&tmA, A, (uint64_t)p.K, (uint64_t)p.M, (uint64_t)lda * 2, BK, BM, 2, true);
  else    rc = make_tmap_2d(&tmA, A, (uint64_t)p.M, (uint64_t)p.K, (uint64_t)lda * 2, 64, BK, 2, true);
  if (rc) return rc;
  if (BK_) rc = make_tmap_2d(&tmB, B, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)ldb * 2, BK, BNH, 2, true);
  else     rc = make_tmap_2d(&tmB, B, (uint64_t)p.N, (uint64_t)p.K, (uint64_t)ldb * 2, 64, BK, 2, true);
  if (rc) return rc;
  CUtensorMap tmOwn = tmA;
  if (COMM == COMM_AG) {
    rc = make_tmap_2d(&tmOwn, cp.x_local, (uint64_t)p.K, (uint64_t)cp.rows_per_shard, (uint64_t)cp.x_ld * 2, BK, BM, 2, true);
    if (rc) return rc;
  }
  p.tiles_m = (p.M + 2 * BM - 1) / (2 * BM); p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  int sms = sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  int clusters = sms / 2;
  if (clusters < 1) clusters = 1;
  const int work = (p.sym_lower ? p.tiles_m * (p.tiles_m + 1) / 2 : tiles) * (p.ksplit > 1 ? p.ksplit : 1);
  if (COMM != COMM_AG && work < clusters) clusters = work;     // AG: copy clusters + GEMM clusters, all co-resident
  auto kern = gemm_bf16_2sm_kernel<AK, BK_, COMM>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, COMM == COMM_RS ? SMEM_RS : SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  kern<<<2 * clusters, THREADS, COMM == COMM_RS ? SMEM_RS : SMEM, stream>>>(tmA, tmB, p, cp, tmOwn);
  return (int)cudaGetLastError();
}

}  // namespace sm2

// C[i][j] = C[j][i] for j > i (bf16, n x n, pitch ldc): fills the tiles a symmetric-output GEMM skipped.
__global__ void symmetrize_lower_kernel(__nv_bfloat16* __restrict__ C, int n, long long ldc) {
  __shared__ __nv_bfloat16 tile[32][34];
  const int bi = blockIdx.y, bj = blockIdx.x;             // source block (rows bi*32.., cols bj*32..) with bj <= bi
  if (bj > bi) return;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    const int i = bi * 32 + r, j = bj * 32 + tx;
    tile[r][tx] = (i < n && j < n) ? C[(long long)i * ldc + j] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int i = bj * 32 + r, j = bi * 32 + tx;          // destination element (i, j) = source (j, i)
    if (i < n && j < n && j > i) C[(long long)i * ldc + j] = tile[tx][r];
  }
}

bool gemm_2sm_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("HIPPO_GEMM_2SM"); v = (e && e[0] == '0') ? 0 : 1; }
  return v == 1;
}

int launch_gemm_2sm(const void* A, const void* B, int layout, long long lda, long long ldb, const GemmParams& p,
                    int max_ctas, cudaStream_t stream) {
  CommParams cp = {};
  switch (layout) {
    case 0: return sm2::launch<true, true, COMM_NONE>(A, B, lda, ldb, p, max_ctas, cp, stream);
    case 1: return sm2::launch<true, false, COMM_NONE>(A, B, lda, ldb, p, max_ctas, cp, stream);
    case 2: return sm2::launch<false, false, COMM_NONE>(A, B, lda, ldb, p, max_ctas, cp, stream);
    case 3: return sm2::launch<false, true, COMM_NONE>(A, B, lda, ldb, p, max_ctas, cp, stream);
  }
  return -1;
}

// All-gather -> GEMM on the CTA-pair kernel (layout 0: B stored [N, K]; 1: B stored [K, N]); cp as for the one-CTA kernel,
// with comm_ctas even and rows_per_shard a multiple of 256.
int launch_allgather_gemm_2sm(const void* A, const void* B, int layout, long long lda, long long ldb, const GemmParams& p,
                              const CommParams& cp, cudaStream_t stream) {
  if (layout == 0) return sm2::launch<true, true, COMM_AG>(A, B, lda, ldb, p, 0, cp, stream);
  if (layout == 1) return sm2::launch<true, false, COMM_AG>(A, B, lda, ldb, p, 0, cp, stream);
  return -1;
}

// GEMM -> reduce-scatter on the CTA-pair kernel (same layouts); rows_per_shard a multiple of 256.
int launch_gemm_reduce_scatter_2sm(const void* A, const void* B, int layout, long long lda, long long ldb,
                                   const GemmParams& p, const CommParams& cp, cudaStream_t stream) {
  if (layout == 0) return sm2::launch<true, true, COMM_RS>(A, B, lda, ldb, p, 0, cp, stream);
  if (layout == 1) return sm2::launch<true, false, COMM_RS>(A, B, lda, ldb, p, 0, cp, stream);
  return -1;
}

// Logits GEMM of the linear + cross-entropy head (C = A B^T, A [M, K], B [N, K], C bf16) with the EPI_LCE epilogue.
int launch_gemm_lce_2sm(const void* A, const void* B, long long lda, long long ldb, const GemmParams& p, cudaStream_t stream) {
  CommParams cp = {};
  return sm2::launch<true, true, EPI_LCE>(A, B, lda, ldb, p, 0, cp, stream);
}

}  // namespace hippo

// Logits of one token chunk with their softmax statistics from the GEMM epilogue.
//   C[M, N] (bf16, pitch ldc)  = A[M, K] B[N, K]^T
//   part[ceil(N / 256)][M]     = per 256-column tile: (max, sum of exp(z - max)) of the row's stored (bf16) logits
//   tz[M]                      = stored logit at column target[row]; rows with target[row] < 0 are left untouched
// target[row] must be -1 or a column in [0, N).
extern "C" int hippo_gemm_bf16_lce(const void* A, const void* B, void* C, float* part, const long long* target, float* tz,
                                   int M, int N, int K, long long lda, long long ldb, long long ldc, void* stream) {
  using namespace hippo;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -2;
  if ((ldc % 8) || ((uintptr_t)C & 15) || ((uintptr_t)part & 7) || !part || !target || !tz) return -3;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = 0; p.accumulate = 0; p.alpha = 1.f;
  p.Cin = nullptr; p.ldcin = 0; p.beta = 0.f; p.tiles_m = p.tiles_n = 0; p.sym_lower = 0; p.ksplit = 0;
  p.lce_part = (float2*)part; p.lce_target = target; p.lce_tz = tz;
  return launch_gemm_lce_2sm(A, B, lda, ldb, p, (cudaStream_t)stream);
}

// Explicit entry point of the CTA-pair kernel (tests and benches compare it with the one-CTA kernel).
// layout code: 0 = NT (A[M,K], B[N,K]); 1 = NN (A[M,K], B[K,N]); 2 = TN (A[K,M], B[K,N]); 3 = TT (A[K,M], B[N,K])
extern "C" int hippo_gemm_bf16_2sm(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K,
                                   long long lda, long long ldb, long long ldc, long long ldcin, int layout,
                                   int out_fp32, int accumulate, float alpha, float beta, void* stream) {
  using namespace hippo;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -2;
  if ((out_fp32 ? (ldc % 4) : (ldc % 8)) || ((uintptr_t)C & 15)) return -3;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate; p.alpha = alpha;
  p.Cin = Cin; p.ldcin = ldcin; p.beta = beta; p.tiles_m = p.tiles_n = 0; p.sym_lower = 0; p.ksplit = 0;
  return launch_gemm_2sm(A, B, layout, lda, ldb, p, 0, (cudaStream_t)stream);
}

// out (+)= alpha * sum over the ksplit partial planes of the fp32 workspace [ksplit][M][N]
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int ksplit, long long plane, void* out, int out_fp32,
                                     long long ldo, int N, int accumulate, float alpha, long long n) {
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    float4 a = *(const float4*)(ws + i);
    for (int s = 1; s < ksplit; ++s) {
      const float4 b = *(const float4*)(ws + s * plane + i);
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    a.x *= alpha; a.y *= alpha; a.z *= alpha; a.w *= alpha;
    const long long r = i / N; const int c = (int)(i % N);          // N % 4 == 0: the four elements share a row
    if (out_fp32) {
      float4* o = (float4*)((float*)out + r * ldo + c);
      if (accumulate) { const float4 v = *o; a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }
      *o = a;
    } else {
      __nv_bfloat162* o = (__nv_bfloat162*)((__nv_bfloat16*)out + r * ldo + c);
      if (accumulate) {
        const float2 v0 = __bfloat1622float2(o[0]), v1 = __bfloat1622float2(o[1]);
        a.x += v0.x; a.y += v0.y; a.z += v1.x; a.w += v1.y;
      }
      o[0] = __floats2bfloat162_rn(a.x, a.y); o[1] = __floats2bfloat162_rn(a.z, a.w);
    }
  }
}

// Split-K product for outputs with too few 256x256 tiles to fill the GPU (weight gradients of narrow projections with
// a contraction over tens of thousands of tokens): work item = (tile, K slice); partial products go to `workspace`
// (fp32, ksplit * M * N elements, provided by the caller), then one reduction pass writes C (+= when accumulate).
// Deterministic: the slices are summed in a fixed order.
extern "C" int hippo_gemm_bf16_splitk(const void* A, const void* B, void* C, float* workspace, int M, int N, int K,
                                      long long lda, long long ldb, long long ldc, int layout, int out_fp32,
                                      int accumulate, float alpha, int ksplit, void* stream) {
  using namespace hippo;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || (N % 4) || ksplit < 2) return -2;
  if ((out_fp32 ? (ldc % 4) : (ldc % 8)) || ((uintptr_t)C & 15) || ((uintptr_t)workspace & 15)) return -3;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.C = workspace; p.ldc = N; p.out_fp32 = 1; p.accumulate = 0; p.alpha = 1.f;
  // every slice must own at least one k-block (an empty slice would publish an accumulator nobody wrote)
  const int kblocks = (K + sm2::BK - 1) / sm2::BK;
  if (ksplit > kblocks) ksplit = kblocks;
  const int kb_per = (kblocks + ksplit - 1) / ksplit;
  ksplit = (kblocks + kb_per - 1) / kb_per;
  p.Cin = nullptr; p.ldcin = 0; p.beta = 0.f; p.tiles_m = p.tiles_n = 0; p.sym_lower = 0; p.ksplit = ksplit;
  int rc = launch_gemm_2sm(A, B, layout, lda, ldb, p, 0, (cudaStream_t)stream);
  if (rc) return rc;
  const long long n = (long long)M * N;
  unsigned grid = (unsigned)((n / 4 + 255) / 256); if (grid > 1184) grid = 1184; if (grid == 0) grid = 1;
  splitk_reduce_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(workspace, ksplit, n, C, out_fp32, ldc, N, accumulate, alpha, n);
  return (int)cudaGetLastError();
}

// Symmetric product (C = C^T by construction, e.g. X X^T or S S + S with S symmetric), bf16 n x n output: only the
// tiles on or below the diagonal are computed, then mirrored. Same arguments as hippo_gemm_bf16_2sm otherwise.
extern "C" int hippo_gemm_bf16_sym(const void* A, const void* B, void* C, const void* Cin, int n, int K, long long lda,
                                   long long ldb, long long ldc, long long ldcin, int layout, float alpha, float beta,
                                   void* stream) {
  using namespace hippo;
  if (n <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15) || (ldc % 8) || ((uintptr_t)C & 15)) return -2;
  GemmParams p;
  p.M = n; p.N = n; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = 0; p.accumulate = 0; p.alpha = alpha;
  p.Cin = Cin; p.ldcin = ldcin; p.beta = beta; p.tiles_m = p.tiles_n = 0; p.sym_lower = 1; p.ksplit = 0;
  int rc = launch_gemm_2sm(A, B, layout, lda, ldb, p, 0, (cudaStream_t)stream);
  if (rc) return rc;
  const unsigned nb = (unsigned)((n + 31) / 32);
  symmetrize_lower_kernel<<<dim3(nb, nb), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)C, n, ldc);
  return (int)cudaGetLastError();
}
