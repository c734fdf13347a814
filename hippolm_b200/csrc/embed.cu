// Vocab-parallel embedding over peer memory.
//
// Forward: every rank needs the embeddings of ITS sequence-parallel token shard. The row of token id v lives on rank
// v / Vl (vocabulary shards of Vl rows); the kernel reads it straight from that rank's weight mirror with plain peer
// loads (NVLink through NVSwitch) and writes the [T/w, D] shard. Only the rows that are needed cross the link:
// T/w * D * 2 bytes per rank, 1/w of what a lookup of all T tokens followed by a reduce-scatter moves.
// Backward: rank r owns dW of its vocabulary rows; it pulls the output-gradient rows of the tokens whose id falls in its
// range from the gradient mirror of the rank whose token shard holds them and accumulates in fp32 (atomicAdd: several
// tokens may share an id). With one rank both kernels are a plain gather / scatter-add of local memory.
// The reference does an all-reduce of a masked full lookup (src/models/tp_model/embed.py:44-61).
#include "sm100.cuh"

namespace hippo {
typedef __nv_bfloat16 bf16;
struct PeerPtrs { const void* p[8]; };

// ids: [n] token ids of this rank's token shard; shards.p[r]: bf16 [Vl, D] weight (mirror) of rank r; out: [n, D] bf16.
// One warp per token row; ids outside [0, world * Vl) give a zero row.
__global__ void embed_gather_kernel(const long long* __restrict__ ids, PeerPtrs shards, int world, int Vl, int D,
                                    bf16* __restrict__ out, long long n) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (long long t = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); t < n; t += (long long)gridDim.x * wpb) {
    const long long id = ids[t];
    (void)HIPPO_IN_BOUNDS(id, (long long)world * Vl, 1);       // debug build: an id outside the vocabulary is recorded
    const int owner = (id >= 0 && id < (long long)world * Vl) ? (int)(id / Vl) : -1;
    uint4* dst = (uint4*)(out + t * D);
    if (owner < 0) {
      for (int v = lane; v < D / 8; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* src = (const uint4*)((const bf16*)shards.p[owner] + (id - (long long)owner * Vl) * D);
    // four independent 16-byte loads in flight per lane (peer loads have microsecond latency)
    for (int v0 = lane; v0 < D / 8; v0 += 128) {
      uint4 tmp[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) if (v0 + 32 * j < D / 8) tmp[j] = src[v0 + 32 * j];
#pragma unroll
      for (int j = 0; j < 4; ++j) if (v0 + 32 * j < D / 8) dst[v0 + 32 * j] = tmp[j];
    }
  }
}

// ids: [T] ids of ALL tokens; grads.p[r]: bf16 [T / world, D] output gradient (mirror) of rank r's token shard;
// dw: fp32 [Vl, D] (+=) for the vocabulary rows [v0, v0 + Vl). One warp per token; tokens of other shards are skipped.
__global__ void embed_grad_kernel(const long long* __restrict__ ids, PeerPtrs grads, int world, long long rows_per_rank,
                                  long long v0, int Vl, int D, float* __restrict__ dw, long long T) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (long long t = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += (long long)gridDim.x * wpb) {
    (void)HIPPO_IN_BOUNDS(ids[t], (long long)world * Vl, 2);
    const long long local = ids[t] - v0;
    if (local < 0 || local >= Vl) continue;
    const int src_rank = (int)(t / rows_per_rank);
    if (src_rank >= world) continue;
    const uint4* src = (const uint4*)((const bf16*)grads.p[src_rank] + (t - (long long)src_rank * rows_per_rank) * D);
    float* dst = dw + local * D;
    for (int v = lane; v < D / 8; v += 32) {
      const uint4 x = src[v];
      const __nv_bfloat162* h = (const __nv_bfloat162*)&x;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        atomicAdd(dst + v * 8 + 2 * e, f.x);
        atomicAdd(dst + v * 8 + 2 * e + 1, f.y);
      }
    }
  }
}
}  // namespace hippo

using namespace hippo;

extern "C" int hippo_embed_gather(const long long* ids, const void* const* shard_ptrs, int world, int Vl, int D, void* out,
                                  long long n, void* stream) {
  if (n <= 0) return 0;
  if (world < 1 || world > 8 || D % 8) return -1;
  PeerPtrs pp = {};
  for (int r = 0; r < world; ++r) pp.p[r] = shard_ptrs[r];
  const unsigned grid = (unsigned)((n + 7) / 8 < 2368 ? (n + 7) / 8 : 2368);
  embed_gather_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(ids, pp, world, Vl, D, (bf16*)out, n);
  return (int)cudaGetLastError();
}

extern "C" int hippo_embed_grad(const long long* ids, const void* const* grad_ptrs, int world, long long rows_per_rank,
                                long long v0, int Vl, int D, float* dw, long long T, void* stream) {
  if (T <= 0) return 0;
  if (world < 1 || world > 8 || D % 8 || rows_per_rank <= 0) return -1;
  PeerPtrs pp = {};
  for (int r = 0; r < world; ++r) pp.p[r] = grad_ptrs[r];
  const unsigned grid = (unsigned)((T + 7) / 8 < 2368 ? (T + 7) / 8 : 2368);
  embed_grad_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(ids, pp, world, rows_per_rank, v0, Vl, D, dw, T);
  return (int)cudaGetLastError();
}
