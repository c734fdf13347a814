// Persistent warp-specialised bf16 GEMM on tcgen05 tensor cores (sm_100a).
//
//   C[M,N] = op(A) * op(B)   fp32 accumulate in TMEM, bf16 or fp32 output
//   A_KMAJOR: A stored [M, K] (contraction contiguous)   else stored [K, M]
//   B_KMAJOR: B stored [N, K] (contraction contiguous)   else stored [K, N]
//
// One CTA per SM, 192 threads: warp 0 = TMA producer, warp 1 = MMA issuer (one elected thread) and
// TMEM owner, warps 2..5 = epilogue (each reads its own 32 TMEM lanes). 128x256 output tile, K in
// slabs of 64 (one 128-byte swizzle atom), 4 smem stages, two TMEM accumulators so the epilogue of
// tile i overlaps the main loop of tile i+1. All loads are plain (non-multicast) TMA.
// Replaces the reference's cuBLAS calls behind F.linear / torch.mm (qkv_proj, o_proj, FFN, LCE).
#include "sm100.cuh"
#include "host_utils.h"
#include "gemm_params.h"
#include "gemm_comm.cuh"
#include <stdlib.h>

namespace hippo {

__device__ Status g_status = {0, 0, 0, 0};

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int GEMM_SMEM_RS = 3 * STAGE_BYTES + 4 * 32 * 512 + 1024 + 256;

// CommParams, the peer-counter helpers and the all-gather copy role are shared with the CTA-pair kernel: gemm_comm.cuh

template <bool A_KMAJOR, bool B_KMAJOR, int COMM>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p,
                 const __grid_constant__ CommParams cp, const __grid_constant__ CUtensorMap tmOwn) {
  // GEMM->RS trades one pipeline stage for a 64 KB epilogue staging area (coalesced 512-byte remote stores)
  constexpr int NST = (COMM == COMM_RS) ? 3 : STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* epi_stage = smem + 3 * STAGE_BYTES;                 // only used by COMM_RS: 4 warps x [32][512 B]
  uint64_t* full = (uint64_t*)(smem + ((COMM == COMM_RS) ? 3 * STAGE_BYTES + 4 * 32 * 512 : STAGES * STAGE_BYTES));
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = (uint32_t*)(tempty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], 4); }
    fence_barrier_init();
    prefetch_tmap(&tmA); prefetch_tmap(&tmB);
    if (COMM == COMM_AG) prefetch_tmap(&tmOwn);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int first_cta = (COMM == COMM_AG) ? cp.comm_ctas : 0;
  const int n_gemm_ctas = gridDim.x - first_cta;
  const int bid = (int)blockIdx.x - first_cta;

  // grouped rasterisation: 8 row-blocks share each column-block sweep so A/B tiles stay hot in L2.
  // With a fused collective the row-blocks are walked shard by shard: AG in arrival order
  // (own, rank-1, rank-2, ...), RS remote owners first (rank+1, ...), own rows last.
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int GROUP = 8;
    int tiles_m = p.tiles_m, base_m = 0;
    if (COMM != COMM_NONE) {
      const int tms = cp.rows_per_shard / BM;            // row-blocks per shard
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
    // ---- copy role, driven by ONE thread with bulk async copies (TMA): a chunk of the local shard is read into shared
    // memory once and stored from there into the gathered buffer of every peer (7 stores per local read at 8 ranks),
    // through a ring of 4 buffers with the loads two chunks ahead of the stores. The shard travels in 128-row blocks;
    // once every store of a block has completed, the block's arrival counter is released on each peer, so consumers
    // start on the first blocks of a remote shard while the rest is still in flight. Own tiles read x_local in place
    // (tmOwn); a caller that needs the complete gathered buffer afterwards copies its own rows in with a device copy.
    if (threadIdx.x == 0) ag_copy_role<STAGE_BYTES, BM, STAGES>(smem, full, cp, p.K, (int)blockIdx.x);
  } else

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      int last_tm = -1;
      for (int t = bid; t < num_tiles && ok; t += n_gemm_ctas) {
        int tm, tn; tile_coord(t, tm, tn);
        const int own_lo = cp.rank * (cp.rows_per_shard / BM), own_hi = own_lo + cp.rows_per_shard / BM;
        const bool own_tile = (COMM == COMM_AG) && tm >= own_lo && tm < own_hi;
        if (COMM == COMM_AG && !own_tile) {
          if (tm != last_tm) {                               // one acquire per new row block (tm is block-indexed)
            ok = wait_counter(cp.flag_peer[cp.rank] + tm, cp.target, cp.wait_cycles, tm);
            asm volatile("fence.proxy.async;" ::: "memory");     // remote generic-proxy writes -> TMA reads
            last_tm = tm;
            if (!ok) break;
          }
        }
        for (int kb = 0; kb < kblocks && ok; ++kb, ++it) {
          int s = it % NST; uint32_t ph = (it / NST) & 1;
          ok = mbar_wait(&empty[s], ph ^ 1, kWaitSmemEmpty, it);
          if (!ok) break;
          uint8_t* sa = smem + s * STAGE_BYTES; uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          if (COMM == COMM_AG && own_tile) {
            tma_load_2d(sa, &tmOwn, &full[s], kb * BK, (tm - own_lo) * BM);
          } else if (A_KMAJOR) {
            tma_load_2d(sa, &tmA, &full[s], kb * BK, tm * BM);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tmA, &full[s], tm * BM + j * 64, kb * BK);
          }
          if (B_KMAJOR) {
            tma_load_2d(sb, &tmB, &full[s], kb * BK, tn * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tmB, &full[s], tn * BN + j * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(BM, BN, 1, A_KMAJOR ? 0 : 1, B_KMAJOR ? 0 : 1);
      int it = 0, tl = 0;
      bool ok = true;
      for (int t = bid; t < num_tiles && ok; t += n_gemm_ctas, ++tl) {
        int acc = tl & 1; uint32_t aph = (tl >> 1) & 1;
        ok = mbar_wait(&tempty[acc], aph ^ 1, kWaitTmemEmpty, tl);
        if (!ok) break;
        tc_fence_after();
        uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          int s = it % NST; uint32_t ph = (it / NST) & 1;
          ok = mbar_wait(&full[s], ph, kWaitTmaFull, it);
          if (!ok) break;
          tc_fence_after();
          uint32_t sa = smem_u32(smem + s * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t ad = A_KMAJOR ? make_smem_desc(sa + k * 32, 16, 1024) : make_smem_desc(sa + k * 2048, 8192, 1024);
            uint64_t bd = B_KMAJOR ? make_smem_desc(sb + k * 32, 16, 1024) : make_smem_desc(sb + k * 2048, 8192, 1024);
            mma_f16_ss(d_tmem, ad, bd, idesc, (kb | k) ? 1u : 0u);
          }
          tc_commit(&empty[s]);
        }
        if (ok) tc_commit(&tfull[acc]);
      }
    }
  } else {
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    int tl = 0;
    int rs_pending = 0;                     // COMM_RS: tiles of the current owner shard stored but not yet released
    bool ok = true;
    for (int t = bid; t < num_tiles && ok; t += n_gemm_ctas, ++tl) {
      int tm, tn; tile_coord(t, tm, tn);
      int acc = tl & 1; uint32_t aph = (tl >> 1) & 1;
      ok = mbar_wait(&tfull[acc], aph, kWaitTmemFull, tl);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      if (COMM == COMM_RS) {
        // partial tile -> staging slot [this rank] of the rank that owns these rows. The warp first lays its
        // 32 x 256 slab out in shared memory, then every store instruction writes one contiguous 512-byte row.
        uint4* slab = (uint4*)(epi_stage + (warp - 2) * 32 * 512);          // [32 rows][32 x 16 B]
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
            const int piece = (c + j) / 8;                                   // 16-byte piece within the row
            slab[lane * 32 + (piece ^ (lane & 31))] = v;                     // xor swizzle: conflict-free both ways
          }
        }
        __syncwarp();
        const int row_base = tm * BM + q * 32;
        const int owner = row_base / cp.rows_per_shard;
        const int ncols = min(BN, p.N - tn * BN);                            // multiple of 8
        __nv_bfloat16* dst0 = (__nv_bfloat16*)cp.buf_peer[owner] +
                              ((long long)cp.rank * cp.rows_per_shard + (row_base - owner * cp.rows_per_shard)) * p.N + tn * BN;
#pragma unroll 4
        for (int rr = 0; rr < 32; ++rr) {
          if (row_base + rr < p.M && lane * 8 < ncols)
            *(uint4*)(dst0 + (long long)rr * p.N + lane * 8) = slab[rr * 32 + (lane ^ (rr & 31))];
        }
        __syncwarp();
      } else
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        EpiPrefetch pre;
        const int col0 = tn * BN + c;
        tmem_ld_32x32(taddr + c, r);
        epi_prefetch(p, row, col0, pre);          // addends travel while the TMEM load completes
        tc_wait_ld();
        epi_store(p, r, row, col0, pre);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);           // the accumulator is free before any remote round trip
      if (COMM == COMM_RS) {
        // one fence + counter release per OWNER SHARD (the owner reduces only after a source's last tile anyway)
        const int owner = (tm * BM) / cp.rows_per_shard;
        ++rs_pending;
        const int tnext = t + n_gemm_ctas;
        int owner_next = -1;
        if (tnext < num_tiles) { int tm2, tn2; tile_coord(tnext, tm2, tn2); owner_next = (tm2 * BM) / cp.rows_per_shard; }
        if (owner_next != owner) {
          __threadfence_system();
          __syncwarp();
          if (lane == 0) red_release_sys_add(cp.flag_peer[owner] + cp.rank, (uint32_t)rs_pending);
          rs_pending = 0;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
  if (COMM == COMM_RS) {
    // ---- reduction of the rows this rank owns: wait for every source, then sum the staging slots
    if ((int)threadIdx.x < cp.world)
      wait_counter(cp.flag_peer[cp.rank] + threadIdx.x, cp.target, cp.wait_cycles, 100 + threadIdx.x);
    __syncthreads();
    const long long nvec = (long long)cp.rows_per_shard * p.N / 8;
    const uint4* stage = (const uint4*)cp.buf_peer[cp.rank];
    uint4* out = (uint4*)cp.out_local;
    const long long stride = (long long)gridDim.x * GEMM_THREADS;
    for (long long v0 = (long long)blockIdx.x * GEMM_THREADS + threadIdx.x; v0 < nvec; v0 += stride * 4) {
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

// addend of the next plain launch (set by hippo_gemm_bf16_ex, cleared after use)
static thread_local const void* g_cin = nullptr;
static thread_local long long g_ldcin = 0;
static thread_local float g_beta = 0.f;

template <bool AK, bool BK_, int COMM>
static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                       long long ldc, int out_fp32, int accumulate, float alpha, int max_ctas, const CommParams& cp,
                       cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  int rc;
  // K-major: global [rows, K], box {64, rows_tile}.  MN-major: global [K, cols], box {64 cols, 64 k-rows}.
  if (AK) rc = make_tmap_2d(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, BM, 2, true);
  else    rc = make_tmap_2d(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, BK, 2, true);
  if (rc) return rc;
  if (BK_) rc = make_tmap_2d(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, BN, 2, true);
  else     rc = make_tmap_2d(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, 64, BK, 2, true);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate; p.alpha = alpha;
  p.Cin = g_cin; p.ldcin = g_ldcin; p.beta = g_beta; p.sym_lower = 0; p.ksplit = 0;
  p.tiles_m = (M + BM - 1) / BM; p.tiles_n = (N + BN - 1) / BN;
  int tiles = p.tiles_m * p.tiles_n;
  int sms = sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  int grid;
  if (COMM == COMM_AG) grid = sms;                                    // copy CTAs + GEMM CTAs, all co-resident
  else if (COMM == COMM_RS) grid = tiles < sms ? tiles : sms;
  else grid = tiles < sms ? tiles : sms;
  CUtensorMap tmOwn = tmA;
  if (COMM == COMM_AG) {
    rc = make_tmap_2d(&tmOwn, cp.x_local, (uint64_t)K, (uint64_t)cp.rows_per_shard, (uint64_t)cp.x_ld * 2, BK, BM, 2, true);
    if (rc) return rc;
  }
  auto kern = gemm_bf16_kernel<AK, BK_, COMM>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         COMM == COMM_RS ? GEMM_SMEM_RS : GEMM_SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  kern<<<grid, GEMM_THREADS, COMM == COMM_RS ? GEMM_SMEM_RS : GEMM_SMEM, stream>>>(tmA, tmB, p, cp, tmOwn);
  return (int)cudaGetLastError();
}

}  // namespace hippo

// layout code: 0 = NT (A[M,K], B[N,K]); 1 = NN (A[M,K], B[K,N]); 2 = TN (A[K,M], B[K,N]); 3 = TT (A[K,M], B[N,K])
static int gemm_bf16_dispatch(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                              long long ldb, long long ldc, int layout, int out_fp32, int accumulate,
                              float alpha, int max_ctas, void* stream, bool allow_pair) {
  using namespace hippo;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || ((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -2;
  if ((out_fp32 ? (ldc % 4) : (ldc % 8)) || ((uintptr_t)C & 15)) return -3;
  cudaStream_t s = (cudaStream_t)stream;
  if (allow_pair && M > 128 && layout >= 0 && layout <= 3 && gemm_2sm_enabled()) {
    // CTA-pair kernel (256x256 tiles over two SMs): half the shared-memory operand traffic per SM
    GemmParams p;
    p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate; p.alpha = alpha;
    p.Cin = g_cin; p.ldcin = g_ldcin; p.beta = g_beta; p.tiles_m = p.tiles_n = 0; p.sym_lower = 0; p.ksplit = 0;
    return launch_gemm_2sm(A, B, layout, lda, ldb, p, max_ctas, s);
  }
  CommParams cp = {};
  switch (layout) {
    case 0: return launch_gemm<true, true, COMM_NONE>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, alpha, max_ctas, cp, s);
    case 1: return launch_gemm<true, false, COMM_NONE>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, alpha, max_ctas, cp, s);
    case 2: return launch_gemm<false, false, COMM_NONE>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, alpha, max_ctas, cp, s);
    case 3: return launch_gemm<false, true, COMM_NONE>(A, B, C, M, N, K, lda, ldb, ldc, out_fp32, accumulate, alpha, max_ctas, cp, s);
  }
  return -1;
}

extern "C" int hippo_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                               long long ldb, long long ldc, int layout, int out_fp32, int accumulate,
                               float alpha, int max_ctas, void* stream) {
  return gemm_bf16_dispatch(A, B, C, M, N, K, lda, ldb, ldc, layout, out_fp32, accumulate, alpha, max_ctas, stream, true);
}

// The one-CTA kernel regardless of size (tests and benches compare the two kernels).
extern "C" int hippo_gemm_bf16_1sm(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                   long long ldb, long long ldc, int layout, int out_fp32, int accumulate,
                                   float alpha, int max_ctas, void* stream) {
  return gemm_bf16_dispatch(A, B, C, M, N, K, lda, ldb, ldc, layout, out_fp32, accumulate, alpha, max_ctas, stream, false);
}

// All-gather -> GEMM.  x_local: [rows_per_shard, K] bf16 (pitch x_ld). xg_ptrs[r]: rank r's gathered buffer
// [world*rows_per_shard, K] (peer-mapped symmetric memory, own entry = local). flag_ptrs[r]: rank r's counters
// [world]. Computes C[world*rows_per_shard, N] = gathered(x) * op(B); layout 0: B stored [N, K]; 1: B stored [K, N].
// flag_ptrs[r]: rank r's counters [world * rows_per_shard/128]; `target` = number of calls made on them (this one included).
extern "C" int hippo_allgather_gemm_bf16(const void* x_local, long long x_ld, void* const* xg_ptrs,
                                         void* const* flag_ptrs, int world, int rank, int rows_per_shard,
                                         const void* B, long long ldb, void* C, long long ldc, int N, int K, int layout,
                                         int comm_ctas, unsigned target, long long wait_cycles, void* stream) {
  using namespace hippo;
  if (world < 1 || world > MAX_RANKS || rows_per_shard % BM || (K % 8) || (N % 8)) return -2;
  CommParams cp = {};
  cp.world = world; cp.rank = rank; cp.rows_per_shard = rows_per_shard; cp.comm_ctas = comm_ctas;
  cp.target = target; cp.wait_cycles = wait_cycles > 0 ? wait_cycles : kWaitCycles;
  cp.x_local = x_local; cp.x_ld = x_ld;
  for (int r = 0; r < world; ++r) { cp.buf_peer[r] = xg_ptrs[r]; cp.flag_peer[r] = (uint32_t*)flag_ptrs[r]; }
  const int M = world * rows_per_shard;
  const void* A = xg_ptrs[rank];
  cudaStream_t s = (cudaStream_t)stream;
  static int pair = -1;
  if (pair < 0) { const char* e = getenv("HIPPO_FUSED_PAIR"); pair = (e && e[0] == '0') ? 0 : 1; }
  if (pair && gemm_2sm_enabled() && rows_per_shard % 256 == 0 && (layout == 0 || layout == 1)) {
    // CTA-pair kernel: 256x256 tiles over two SMs, copy role in whole clusters
    cp.comm_ctas = (comm_ctas + 1) & ~1;
    GemmParams p;
    p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.out_fp32 = 0; p.accumulate = 0; p.alpha = 1.f;
    p.Cin = nullptr; p.ldcin = 0; p.beta = 0.f; p.tiles_m = p.tiles_n = 0; p.sym_lower = 0; p.ksplit = 0;
    return launch_allgather_gemm_2sm(A, B, layout, K, ldb, p, cp, s);
  }
  if (layout == 0) return launch_gemm<true, true, COMM_AG>(A, B, C, M, N, K, K, ldb, ldc, 0, 0, 1.f, 0, cp, s);
  if (layout == 1) return launch_gemm<true, false, COMM_AG>(A, B, C, M, N, K, K, ldb, ldc, 0, 0, 1.f, 0, cp, s);
  return -1;
}

// GEMM -> reduce-scatter.  A: [world*rows_per_shard, K] local bf16; partial C tiles are stored into the staging
// slot [rank] of the owning rank (stage_ptrs[r]: [world][rows_per_shard, N] bf16 on rank r), then every rank sums its
// own slots into out_local [rows_per_shard, N]. `target` = calls so far * (rows_per_shard/128) * ceil(N/256) * 4.
extern "C" int hippo_gemm_reduce_scatter_bf16(const void* A, long long lda, const void* B, long long ldb,
                                              void* const* stage_ptrs, void* const* flag_ptrs, int world, int rank,
                                              int rows_per_shard, void* out_local, int N, int K, int layout,
                                              unsigned target, long long wait_cycles, void* stream) {
  using namespace hippo;
  if (world < 1 || world > MAX_RANKS || rows_per_shard % BM || (K % 8) || (N % 8)) return -2;
  CommParams cp = {};
  cp.world = world; cp.rank = rank; cp.rows_per_shard = rows_per_shard; cp.target = target;
  cp.wait_cycles = wait_cycles > 0 ? wait_cycles : kWaitCycles;
  for (int r = 0; r < world; ++r) { cp.buf_peer[r] = stage_ptrs[r]; cp.flag_peer[r] = (uint32_t*)flag_ptrs[r]; }
  cp.out_local = out_local;
  const int M = world * rows_per_shard;
  cudaStream_t s = (cudaStream_t)stream;
  static int pair = -1;
  if (pair < 0) { const char* e = getenv("HIPPO_FUSED_PAIR"); pair = (e && e[0] == '0') ? 0 : 1; }
  if (pair && gemm_2sm_enabled() && rows_per_shard % 256 == 0 && (layout == 0 || layout == 1)) {
    GemmParams p;
    p.M = M; p.N = N; p.K = K; p.C = nullptr; p.ldc = N; p.out_fp32 = 0; p.accumulate = 0; p.alpha = 1.f;
    p.Cin = nullptr; p.ldcin = 0; p.beta = 0.f; p.tiles_m = p.tiles_n = 0; p.sym_lower = 0; p.ksplit = 0;
    return launch_gemm_reduce_scatter_2sm(A, B, layout, lda, ldb, p, cp, s);
  }
  if (layout == 0) return launch_gemm<true, true, COMM_RS>(A, B, nullptr, M, N, K, lda, ldb, N, 0, 0, 1.f, 0, cp, s);
  if (layout == 1) return launch_gemm<true, false, COMM_RS>(A, B, nullptr, M, N, K, lda, ldb, N, 0, 0, 1.f, 0, cp, s);
  return -1;
}

// C = alpha * op(A) op(B) + beta * Cin   (bf16 output; Cin may not alias C unless beta-only semantics are acceptable
// per element, which they are: each output element is read once and written once by the same thread)
extern "C" int hippo_gemm_bf16_ex(const void* A, const void* B, void* C, const void* Cin, int M, int N, int K,
                                  long long lda, long long ldb, long long ldc, long long ldcin, int layout, float alpha,
                                  float beta, void* stream) {
  hippo::g_cin = Cin; hippo::g_ldcin = ldcin; hippo::g_beta = beta;
  int rc = hippo_gemm_bf16(A, B, C, M, N, K, lda, ldb, ldc, layout, 0, 0, alpha, 0, stream);
  hippo::g_cin = nullptr; hippo::g_beta = 0.f;
  return rc;
}

extern "C" int hippo_get_status(int* out4) {
  hippo::Status st;
  cudaError_t e = cudaMemcpyFromSymbol(&st, hippo::g_status, sizeof(st));
  if (e != cudaSuccess) return (int)e;
  out4[0] = st.code; out4[1] = st.detail; out4[2] = st.block; out4[3] = st.count;
  return 0;
}

extern "C" int hippo_clear_status() {
  hippo::Status st = {0, 0, 0, 0};
  return (int)cudaMemcpyToSymbol(hippo::g_status, &st, sizeof(st));
}
