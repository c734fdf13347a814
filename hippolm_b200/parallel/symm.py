"""Symmetric (peer-mapped) memory workspace for the fused compute + collective kernels.

The buffers are allocated with ``torch.distributed._symmetric_memory`` (cuMemCreate + handle exchange
over the TP group); the kernels in ``csrc/gemm_bf16.cu`` only see raw peer pointers:

  gathered[parity]   [T, Kmax] bf16 on every rank   target of the all-gather pushes (AG -> GEMM)
  staging[parity]    [world][T/world, Nmax] bf16     per-source partial tiles (GEMM -> RS)
  gathered_fp4[par]  NVFP4 bytes + scale tiles      target of the quantise-and-push kernel (FP4 AG -> GEMM)
  lce_stats[par]     float4 [world][T]              per-source (max, sum exp, target logit) rows of the LCE head
  counters           uint32 [8][1024]                monotonic arrival counters, one row per (op, parity); AG: one per
                                                     (source rank, 128-row block), RS: one per source rank

A rank can run at most one fused op ahead of its slowest peer (each op needs data from every peer), so
two parities per op type are enough to keep a fast rank's pushes out of a buffer a slow rank still reads.
Every wait inside the kernels is bounded; ``check_status`` raises if one ran out.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops._ext import lib, ptr, stream_ptr, check

_BM, _BN = 128, 256


def _ptr_arr(ptrs) -> C.Array:
    return (C.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


class FusedWorkspace:
    FLAG_ROW = 1024          # counters per (op, parity) row: world * row blocks per shard <= 1024
    N_ROWS = 8

    def __init__(self, mesh, max_tokens: int, max_width: int, dtype=torch.bfloat16, comm_ctas: int = 16,
                 wait_cycles: int = 0):
        import torch.distributed._symmetric_memory as symm_mem
        assert dtype == torch.bfloat16
        self.mesh, self.world, self.rank = mesh, mesh.tp, mesh.tp_rank
        self.max_tokens, self.max_width = max_tokens, max_width
        self.comm_ctas, self.wait_cycles = comm_ctas, wait_cycles
        dev = mesh.device
        group = mesh.tp_group if mesh.tp_group is not None else dist.group.WORLD
        nbytes = max_tokens * max_width * 2
        self._bufs, self._hdls = [], []

        def alloc(n):
            t = symm_mem.empty(n, dtype=torch.uint8, device=dev)
            h = symm_mem.rendezvous(t, group)
            self._bufs.append(t); self._hdls.append(h)
            return t, [int(p) for p in h.buffer_ptrs]

        self.gathered = [alloc(nbytes) for _ in range(2)]
        self.staging = [alloc(nbytes) for _ in range(2)]
        # NVFP4 gathered activations: [T, K/2] packed | [T/128][K/64][512] scale tiles | 8 tensor scales
        self.gathered_fp4 = [alloc(max_tokens * max_width * 9 // 16 + 256) for _ in range(2)]
        self.lce_rows = max_tokens
        self.lce_stats = [alloc(self.world * max_tokens * 16) for _ in range(2)]
        self.lce_n = 0
        self.flags_t, self.flag_ptrs = alloc(self.N_ROWS * self.FLAG_ROW * 4)
        self.flags_t.zero_()
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)
        self._group = group
        # per counter row (bf16 AG parity 0/1, RS parity 0/1, FP4 AG parity 0/1): the value every counter of the row
        # reaches once all calls made so far have completed, and the row-block count those calls used
        self.targets = [0] * self.N_ROWS
        self.row_blocks = [0] * self.N_ROWS
        self.ag_n = 0
        self.rs_n = 0
        self.fp4_n = 0

    def _row_ptrs(self, row: int) -> List[int]:
        return [p + row * self.FLAG_ROW * 4 for p in self.flag_ptrs]

    def _use_row(self, row: int, blocks: int, increment: int) -> int:
        """Book one call on a counter row and return its target. Every counter of a row must see the same
        increments, so a call that indexes the row differently (another row-block count) first drains the
        group and restarts the row from zero; all ranks take this branch at the same call."""
        if self.row_blocks[row] not in (0, blocks):
            torch.cuda.synchronize(self.mesh.device)
            dist.barrier(group=self._group)
            self.flags_t.view(torch.int32).view(self.N_ROWS, self.FLAG_ROW)[row].zero_()
            torch.cuda.synchronize(self.mesh.device)
            dist.barrier(group=self._group)
            self.targets[row] = 0
        self.row_blocks[row] = blocks
        self.targets[row] = (self.targets[row] + increment) & 0xFFFFFFFF     # the kernels compare modulo 2^32
        return self.targets[row]

    def reset_counters(self) -> None:
        """Collective over the TP group: bring every arrival counter and its host-side target back to zero. Used after a
        bounded wait ran out (a kernel that gave up leaves arrivals missing, and every later call on that counter row
        would wait for them): all ranks drain their streams, meet, clear their counters, and meet again before the
        next fused call."""
        torch.cuda.synchronize(self.mesh.device)
        dist.barrier(group=self._group)
        self.flags_t.zero_()
        torch.cuda.synchronize(self.mesh.device)
        dist.barrier(group=self._group)
        self.targets = [0] * self.N_ROWS
        self.row_blocks = [0] * self.N_ROWS

    # ------------------------------------------------------------------ all-gather -> GEMM
    def allgather_gemm(self, x: torch.Tensor, weight: torch.Tensor, transpose_w: bool = False,
                       need_gathered: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        """x: [T/w, K] -> (gathered x [T, K] (a view of the workspace, valid until the next-but-one call),
        y [T, N]) with y = gather(x) @ W^T (W: [N, K]) or gather(x) @ W (W: [K, N], transpose_w)."""
        rows, K = x.shape
        N = weight.shape[1] if transpose_w else weight.shape[0]
        T = rows * self.world
        assert rows % _BM == 0 and T * K <= self.max_tokens * self.max_width, "workspace too small / ragged shard"
        assert T // _BM <= self.FLAG_ROW
        x = x.contiguous()
        weight = weight.contiguous()
        par = self.ag_n & 1
        self.ag_n += 1
        row = par
        target = self._use_row(row, rows // _BM, 1)
        buf, ptrs = self.gathered[par]
        y = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
        check(lib().hippo_allgather_gemm_bf16(ptr(x), C.c_longlong(x.stride(0)), _ptr_arr(ptrs), _ptr_arr(self._row_ptrs(row)),
                                              self.world, self.rank, rows, ptr(weight), C.c_longlong(weight.stride(0)),
                                              ptr(y), C.c_longlong(N), N, K, 1 if transpose_w else 0, self.comm_ctas,
                                              C.c_uint(target),
                                              C.c_longlong(self.wait_cycles), stream_ptr()), "allgather_gemm")
        xg = buf[:T * K * 2].view(torch.bfloat16).view(T, K)
        if need_gathered:
            # the kernel reads the own shard in place; complete the gathered view for later users (dW GEMM)
            xg[self.rank * rows:(self.rank + 1) * rows].copy_(x)
        return xg, y

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_reduce_scatter(self, x: torch.Tensor, weight: torch.Tensor, transpose_w: bool = False) -> torch.Tensor:
        """x: [T, K_local] -> reduce_scatter(x @ W^T) [T/w, N] (W: [N, K_local]; transpose_w: W is [K_local, N])."""
        T, K = x.shape
        N = weight.shape[1] if transpose_w else weight.shape[0]
        rows = T // self.world
        assert rows % _BM == 0 and T * N <= self.max_tokens * self.max_width
        x = x.contiguous(); weight = weight.contiguous()
        par = self.rs_n & 1
        self.rs_n += 1
        row = 2 + par
        _, ptrs = self.staging[par]
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=x.device)
        tiles = (rows // _BM) * ((N + _BN - 1) // _BN)
        target = self._use_row(row, 1, tiles * 4)
        check(lib().hippo_gemm_reduce_scatter_bf16(ptr(x), C.c_longlong(x.stride(0)), ptr(weight),
                                                   C.c_longlong(weight.stride(0)), _ptr_arr(ptrs),
                                                   _ptr_arr(self._row_ptrs(row)), self.world, self.rank, rows, ptr(out),
                                                   N, K, 1 if transpose_w else 0, C.c_uint(target),
                                                   C.c_longlong(self.wait_cycles), stream_ptr()), "gemm_reduce_scatter")
        return out

    # ------------------------------------------------------------------ NVFP4: quantise + push -> FP4 GEMM
    def nvfp4_allgather_gemm(self, x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor,
                             global_scale: torch.Tensor, keep_gathered: bool = False):
        """x: [T/w, K] bf16 -> Q(gather(x)) dq(W)^T [T, N]. Each rank quantises its shard with its own tensor scale and
        pushes 0.5625 bytes per element to every peer; the GEMM applies the source rank's scale per row block."""
        from ..ops import fp4_gemm
        rows, K = x.shape
        N = packed.shape[0]
        T = rows * self.world
        if rows % _BM or K % 512 or N % 8 or x.dtype != torch.bfloat16 or T * K > self.max_tokens * self.max_width \
                or T // _BM > self.FLAG_ROW:
            return None, None
        x = x.contiguous()
        par = self.fp4_n & 1
        self.fp4_n += 1
        row = 4 + par
        target = self._use_row(row, rows // _BM, K // 512)
        buf, ptrs = self.gathered_fp4[par]
        gs = torch.empty(1, dtype=torch.float32, device=x.device)
        scratch = torch.empty(1, dtype=torch.float32, device=x.device)
        check(lib().hippo_nvfp4_tensor_scale(ptr(x), C.c_longlong(x.numel()), 1, ptr(scratch), ptr(gs), stream_ptr()),
              "nvfp4_tensor_scale")
        check(lib().hippo_nvfp4_quant_push(ptr(x), C.c_longlong(x.stride(0)), rows, K, ptr(gs), _ptr_arr(ptrs),
                                           _ptr_arr(self._row_ptrs(row)), self.world, self.rank, stream_ptr()),
              "nvfp4_quant_push")
        sfb = fp4_gemm.tile_weight_scales(scales, N, K)
        y = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
        gsw = global_scale.float().contiguous()
        check(lib().hippo_allgather_gemm_nvfp4(ptr(buf), C.c_void_p(self._row_ptrs(row)[self.rank]), self.world, self.rank,
                                               rows, ptr(packed), ptr(sfb), ptr(gsw), ptr(y), C.c_longlong(N), N, K,
                                               C.c_uint(target), C.c_longlong(self.wait_cycles), stream_ptr()),
              "allgather_gemm_nvfp4")
        if keep_gathered:
            # the gathered FP4 activations (packed + scale tiles + per-source tensor scales) for the backward dW
            nbytes = T * K // 2 + T * K // 16 + 32
            return y, buf[:nbytes].clone()
        return y, None

    def nvfp4_dequant_gathered(self, saved: torch.Tensor, T: int, K: int) -> torch.Tensor:
        """bf16 [T, K] view of a gathered FP4 buffer kept by ``nvfp4_allgather_gemm``."""
        out = torch.empty((T, K), dtype=torch.bfloat16, device=saved.device)
        check(lib().hippo_nvfp4_dequant_gathered(ptr(saved), C.c_longlong(T), K, T // self.world, ptr(out), stream_ptr()),
              "nvfp4_dequant_gathered")
        return out

    def nvfp4_gemm_reduce_scatter(self, x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor,
                                  global_scale: torch.Tensor) -> Optional[torch.Tensor]:
        """x: [T, K_local] bf16 -> reduce_scatter(Q(x) dq(W)^T) [T/w, N]; partial tiles leave from the GEMM epilogue."""
        from ..ops import fp4_gemm, nvfp4_cuda
        T, K = x.shape
        N = packed.shape[0]
        rows = T // self.world
        if rows % _BM or T % self.world or K % 256 or N % 8 or x.dtype != torch.bfloat16 \
                or T * N > self.max_tokens * self.max_width:
            return None
        xp, xs, xg = nvfp4_cuda.quantize(x.contiguous())
        sfa, sfb = fp4_gemm.tile_scales(xs, T, K), fp4_gemm.tile_weight_scales(scales, N, K)
        par = self.rs_n & 1
        self.rs_n += 1
        row = 2 + par
        _, ptrs = self.staging[par]
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=x.device)
        tiles = (rows // _BM) * ((N + 127) // 128)
        target = self._use_row(row, 1, tiles * 4)
        gsw = global_scale.float().contiguous()
        check(lib().hippo_gemm_reduce_scatter_nvfp4(ptr(xp), ptr(sfa), ptr(xg), ptr(packed), ptr(sfb), ptr(gsw),
                                                    _ptr_arr(ptrs), _ptr_arr(self._row_ptrs(row)), self.world, self.rank,
                                                    rows, ptr(out), N, K, C.c_uint(target),
                                                    C.c_longlong(self.wait_cycles), stream_ptr()),
              "gemm_reduce_scatter_nvfp4")
        return out

    # ------------------------------------------------------------------ vocab-parallel CE: in-kernel cross-rank softmax
    def lce_stats_push(self, z: torch.Tensor, targets_local: torch.Tensor):
        """Row statistics of this rank's logits shard z[C, V/w] pushed to every rank. Returns the handle for lce_grad_merge."""
        Cr, V = z.shape
        assert Cr <= self.lce_rows and z.dtype == torch.float32 and z.is_contiguous()
        par = self.lce_n & 1
        self.lce_n += 1
        row = 6 + par
        target = self._use_row(row, 1, Cr)
        _, ptrs = self.lce_stats[par]
        tg = targets_local.to(torch.int64).contiguous()
        check(lib().hippo_ce_stats_push(ptr(z), ptr(tg), C.c_longlong(Cr), V, _ptr_arr(ptrs), _ptr_arr(self._row_ptrs(row)),
                                        self.world, self.rank, self.lce_rows, stream_ptr()), "ce_stats_push")
        return (par, row, target, tg)

    def lce_grad_merge(self, handle, z: torch.Tensor, row_weight: torch.Tensor, loss_sum: torch.Tensor) -> torch.Tensor:
        """dz[C, V/w] (bf16) from the merged statistics of all ranks; adds sum(lse - z_target) of weighted rows to loss_sum."""
        par, row, target, tg = handle
        Cr, V = z.shape
        _, ptrs = self.lce_stats[par]
        dz = torch.empty((Cr, V), dtype=torch.bfloat16, device=z.device)
        rw = row_weight.float().contiguous()
        check(lib().hippo_ce_grad_merge(ptr(z), ptr(tg), ptr(rw), ptr(dz), C.c_longlong(Cr), V, ptr(loss_sum), _ptr_arr(ptrs),
                                        _ptr_arr(self._row_ptrs(row)), self.world, self.rank, self.lce_rows,
                                        C.c_uint(target), C.c_longlong(self.wait_cycles), stream_ptr()), "ce_grad_merge")
        return dz

    def lce_part_push(self, part: torch.Tensor, tz: torch.Tensor, tg: torch.Tensor):
        """Statistics from the logits GEMM epilogue (``cuda_ops.lce_logits_stats``): merges the per-tile pairs of every
        row and pushes (max, sum exp, target logit) to every rank. Returns the handle for lce_grad_inplace."""
        tiles_n, Cr = part.shape[0], part.shape[1]
        assert Cr <= self.lce_rows and part.dtype == torch.float32 and part.is_contiguous()
        par = self.lce_n & 1
        self.lce_n += 1
        row = 6 + par
        target = self._use_row(row, 1, Cr)
        _, ptrs = self.lce_stats[par]
        check(lib().hippo_ce_part_merge(ptr(part), ptr(tz), ptr(tg), C.c_longlong(Cr), tiles_n, _ptr_arr(ptrs),
                                        _ptr_arr(self._row_ptrs(row)), self.world, self.rank, self.lce_rows, stream_ptr()),
              "ce_part_merge")
        return (par, row, target, tg)

    def lce_grad_inplace(self, handle, z: torch.Tensor, row_weight: torch.Tensor, loss_sum: torch.Tensor) -> torch.Tensor:
        """Overwrites the bf16 logits z[C, V/w] with dz from the merged statistics of all ranks; adds sum(lse - z_target)
        of weighted rows to loss_sum."""
        par, row, target, tg = handle
        Cr, V = z.shape
        assert z.dtype == torch.bfloat16 and z.is_contiguous() and V % 8 == 0
        _, ptrs = self.lce_stats[par]
        rw = row_weight.float().contiguous()
        check(lib().hippo_ce_grad_inplace(ptr(z), ptr(tg), ptr(rw), C.c_longlong(Cr), V, ptr(loss_sum), _ptr_arr(ptrs),
                                          _ptr_arr(self._row_ptrs(row)), self.world, self.rank, self.lce_rows,
                                          C.c_uint(target), C.c_longlong(self.wait_cycles), stream_ptr()), "ce_grad_inplace")
        return z

    def check_status(self) -> None:
        st = _ext.device_status()
        if st[0] != 0:
            raise RuntimeError(f"a bounded device wait ran out: code={st[0]} detail={st[1]} block={st[2]} count={st[3]}")


class SymmetricMirror:
    """A peer-readable copy of a per-rank tensor (the embedding shard, an output-gradient shard): ``parities`` buffers
    of ``nbytes`` in symmetric memory. ``publish(src, parity)`` copies ``src`` in and runs a barrier over the TP group on
    the current stream, after which every rank may read every rank's buffer of that parity through ``ptrs(parity)``.
    With two parities a rank can publish the next tensor while slower peers still read the previous one."""

    def __init__(self, mesh, nbytes: int, parities: int = 1):
        import torch.distributed._symmetric_memory as symm_mem
        self.mesh = mesh
        self.group = mesh.tp_group if mesh.tp_group is not None else dist.group.WORLD
        self.nbytes = int(nbytes)
        self._bufs, self._ptrs = [], []
        for _ in range(parities):
            t = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=mesh.device)
            h = symm_mem.rendezvous(t, self.group)
            self._bufs.append((t, h))
            self._ptrs.append([int(p) for p in h.buffer_ptrs])
        self._token = torch.zeros(1, device=mesh.device)

    def ptrs(self, parity: int = 0) -> List[int]:
        return self._ptrs[parity]

    def local(self, parity: int = 0) -> torch.Tensor:
        return self._bufs[parity][0]

    def publish(self, src: torch.Tensor, parity: int = 0) -> None:
        raw = src.contiguous().view(torch.uint8).reshape(-1)
        assert raw.numel() <= self.nbytes
        self._bufs[parity][0][:raw.numel()].copy_(raw)
        # stream-ordered barrier: the collective completes on a rank only after every rank has reached it, i.e. after
        # every rank's copy above
        dist.all_reduce(self._token, group=self.group)


def create_workspace(mesh, max_tokens: int, max_width: int, dtype=torch.bfloat16, wait_cycles: int = 0
                     ) -> Optional[FusedWorkspace]:
    if mesh.tp <= 1 or mesh.device.type != "cuda":
        return None
    return FusedWorkspace(mesh, max_tokens, max_width, dtype, wait_cycles=wait_cycles)
