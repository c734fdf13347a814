// Pieces shared by the fused compute + collective modes of the one-CTA and the CTA-pair bf16 GEMM kernels: the
// parameter block, the peer-counter primitives (every spin is bounded) and the all-gather copy role.
#pragma once
#include "sm100.cuh"

namespace hippo {

// Fused collective modes (COMM template parameter of the kernels):
//   COMM_AG  all-gather -> GEMM. The first `comm_ctas` CTAs push this rank's row shard of A into every
//            peer's gathered buffer and bump the peer's arrival counter; GEMM CTAs walk the M tiles in arrival
//            order and their TMA producer waits (bounded) on the counter of the source row block before the first
//            load of that block. Every TMA load reads local memory.
//   COMM_RS  GEMM -> reduce-scatter. The epilogue stores each partial tile into the staging slot of the
//            rank that owns those rows (P2P stores) and bumps that rank's counter; after its last tile
//            every CTA joins the reduction of the local rows (wait for all sources, sum the slots).
//   EPI_LCE  no collective: a plain GEMM whose epilogue also emits per-tile softmax statistics (CTA-pair kernel only; the
//            logits GEMM of the linear + cross-entropy head, see GemmParams::lce_part).
constexpr int COMM_NONE = 0, COMM_AG = 1, COMM_RS = 2, EPI_LCE = 3;
constexpr int MAX_RANKS = 8;

struct CommParams {
  int world, rank;
  int rows_per_shard;                 // AG: rows of A per source rank; RS: rows of C per owner rank
  int comm_ctas;                      // AG: CTAs that copy instead of computing
  uint32_t target;                    // counter value that means "complete for this call"
  long long wait_cycles;              // bound of every spin
  const void* x_local;                // AG: [rows_per_shard, K] bf16 (this rank's shard)
  long long x_ld;                     // AG: row pitch of x_local in elements
  void* buf_peer[MAX_RANKS];          // AG: gathered [world*rows_per_shard, K]; RS: staging [world][rows_per_shard, N]
  uint32_t* flag_peer[MAX_RANKS];     // counters on every rank, indexed by source rank
  void* out_local;                    // RS: [rows_per_shard, N] bf16
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded spin on a monotonic counter written by other GPUs
__device__ __forceinline__ bool wait_counter(const uint32_t* p, uint32_t target, long long limit, int detail) {
  if ((int32_t)(ld_acquire_sys(p) - target) >= 0) return true;
  long long t0 = clock64();
  while ((int32_t)(ld_acquire_sys(p) - target) < 0) {
    if (clock64() - t0 > limit) { report(kWaitPeerFlag, detail); return false; }
    __nanosleep(64);
  }
  return true;
}


// ---- all-gather copy role, driven by ONE thread with bulk async copies (TMA): a chunk of the local shard is read into
// shared memory once and stored from there into the gathered buffer of every peer (7 stores per local read at 8 ranks),
// through a ring of NB buffers of STAGE bytes with the loads two chunks ahead of the stores and up to NB - 2 store groups
// in flight (the transfer is bound by the number of bytes in flight per copy CTA, not by issue rate). The shard travels in
// 128-row blocks; once every store of a block has completed, the block's arrival counter is released on each peer, so
// consumers start on the first blocks of a remote shard while the rest is still in flight. Own tiles read x_local in
// place; a caller that needs the complete gathered buffer afterwards copies its own rows in with a device copy.
// `smem`: NB * STAGE bytes; `full`: NB mbarriers initialised with count 1; `cta`: index of this copy CTA in [0, comm_ctas).
template <int STAGE, int BLOCK_ROWS, int NB>
__device__ __forceinline__ void ag_copy_role(uint8_t* smem, uint64_t* full, const CommParams& cp, int K, int cta) {
  const long long row_bytes = (long long)K * 2;
  const int bps = cp.rows_per_shard / BLOCK_ROWS;                     // 128-row blocks per shard
  int rpc = (int)(STAGE / row_bytes);                                 // rows per chunk (one ring buffer)
  if (rpc > BLOCK_ROWS) rpc = BLOCK_ROWS;
  if (rpc < 1) rpc = 1;
  const int cpb = (BLOCK_ROWS + rpc - 1) / rpc;                       // chunks per block
  const int my_blocks = (bps - cta + cp.comm_ctas - 1) / cp.comm_ctas;
  const int total = my_blocks > 0 ? my_blocks * cpb : 0;
  const bool contiguous = cp.x_ld == (long long)K;
  auto chunk_rows = [&](int c, int& rb, int& r0) {                    // chunk -> (row block, first row in block) -> rows
    rb = cta + (c / cpb) * cp.comm_ctas;
    r0 = (c % cpb) * rpc;
    return min(rpc, BLOCK_ROWS - r0);
  };
  auto load = [&](int c) {
    int rb, r0; const int nr = chunk_rows(c, rb, r0);
    uint8_t* buf = smem + (c % NB) * STAGE;
    const uint8_t* src = (const uint8_t*)cp.x_local + ((long long)rb * BLOCK_ROWS + r0) * cp.x_ld * 2;
    mbar_expect_tx(&full[c % NB], (uint32_t)(nr * row_bytes));
    if (contiguous) {
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem_u32(buf)), "l"(src), "r"((uint32_t)(nr * row_bytes)), "r"(smem_u32(&full[c % NB])) : "memory");
    } else {
      for (int r = 0; r < nr; ++r)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(buf + r * row_bytes)), "l"(src + (long long)r * cp.x_ld * 2), "r"((uint32_t)row_bytes),
                       "r"(smem_u32(&full[c % NB])) : "memory");
    }
  };
  auto release_block = [&](int rb) {
    for (int i = 1; i < cp.world; ++i) {
      const int peer = (cp.rank + i) % cp.world;
      red_release_sys_add(cp.flag_peer[peer] + cp.rank * bps + rb, 1u);
    }
  };
  bool ok = row_bytes <= STAGE && (row_bytes % 16) == 0;
  if (!ok) report(kBadArgument, K);
  if (ok && total > 0) { load(0); if (total > 1) load(1); }
  int released = 0;                                                   // chunks whose blocks have been released so far
  for (int c = 0; ok && c < total; ++c) {
    // stores of chunks <= c + 2 - NB are complete (wait at the end of the previous iteration): the buffer of chunk c + 2,
    // last used by chunk c + 2 - NB, is free
    if (c + 2 < total) load(c + 2);
    ok = mbar_wait(&full[c % NB], (c / NB) & 1, kWaitTmaFull, c);
    if (!ok) break;
    int rb, r0; const int nr = chunk_rows(c, rb, r0);
    const uint8_t* buf = smem + (c % NB) * STAGE;
    const long long off = ((long long)cp.rank * cp.rows_per_shard + (long long)rb * BLOCK_ROWS + r0) * row_bytes;
    for (int i = 1; i < cp.world; ++i) {
      const int peer = (cp.rank + i) % cp.world;
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                   ::"l"((uint8_t*)cp.buf_peer[peer] + off), "r"(smem_u32(buf)), "r"((uint32_t)(nr * row_bytes)) : "memory");
    }
    tma_store_commit();
    tma_store_wait<NB - 3>();                                         // all but the newest NB - 3 groups have completed
    // chunks 0 .. c - (NB - 3) are complete: release every block that ends inside them
    while (released + cpb <= c + 1 - (NB - 3)) { release_block(cta + (released / cpb) * cp.comm_ctas); released += cpb; }
  }
  tma_store_wait<0>();
  if (ok) while (released < total) { release_block(cta + (released / cpb) * cp.comm_ctas); released += cpb; }
}

// CTA-pair all-gather -> GEMM launcher (gemm_bf16_2sm.cu)
struct GemmParams;
int launch_allgather_gemm_2sm(const void* A, const void* B, int layout, long long lda, long long ldb, const GemmParams& p,
                              const CommParams& cp, cudaStream_t stream);
int launch_gemm_reduce_scatter_2sm(const void* A, const void* B, int layout, long long lda, long long ldb,
                                   const GemmParams& p, const CommParams& cp, cudaStream_t stream);

}  // namespace hippo
