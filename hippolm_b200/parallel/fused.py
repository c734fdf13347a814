"""Fused compute + collective kernels over NVSwitch peer memory (entry points).

``setup()`` allocates the symmetric workspace for the current TP group and switches the
sequence-parallel linears from "NCCL then GEMM" to the single-kernel paths in
``csrc/gemm_bf16.cu`` / ``csrc/gemm_fp4.cu`` / ``csrc/lce_fused.cu``. Until it is called (or on CPU) ``enabled()`` is False and the NCCL/gloo
baseline runs.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, Optional, Tuple

import torch

_STATE = {"ws": None}


def enabled() -> bool:
    return _STATE["ws"] is not None


def fits(rows_per_shard: int, tokens: int, width: int) -> bool:
    """Shapes the fused kernels accept: 128-row shards, 8-element columns, inside the workspace."""
    ws = _STATE["ws"]
    return (ws is not None and rows_per_shard % 128 == 0 and width % 8 == 0
            and tokens * width <= ws.max_tokens * ws.max_width)


def setup(mesh, max_tokens: int, max_width: int, dtype=torch.bfloat16, wait_cycles: int = 0) -> bool:
    from . import symm
    ws = symm.create_workspace(mesh, max_tokens, max_width, dtype, wait_cycles=wait_cycles)
    _STATE["ws"] = ws
    return ws is not None


def teardown() -> None:
    _STATE["ws"] = None
    _CHOICE.clear()


def allgather_gemm(x: torch.Tensor, weight: torch.Tensor, transpose_w: bool = False, need_gathered: bool = True
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    return _STATE["ws"].allgather_gemm(x, weight, transpose_w, need_gathered)


def gemm_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, transpose_w: bool = False) -> torch.Tensor:
    return _STATE["ws"].gemm_reduce_scatter(x, weight, transpose_w)


def nvfp4_allgather_gemm(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor,
                         keep_gathered: bool = False):
    """x[T/w, K] bf16 -> (Q(gather(x)) dq(W)^T [T, N], kept gathered FP4 bytes or None) with the FP4 shard exchange
    inside the quantise and GEMM kernels. (None, None) when the workspace / kernel does not cover the shape (the
    caller then runs NCCL + the plain FP4 GEMM)."""
    ws = _STATE["ws"]
    if ws is None:
        return None, None
    return ws.nvfp4_allgather_gemm(x, packed, scales, global_scale, keep_gathered)


def nvfp4_dequant_gathered(saved: torch.Tensor, T: int, K: int) -> torch.Tensor:
    return _STATE["ws"].nvfp4_dequant_gathered(saved, T, K)


def nvfp4_gemm_reduce_scatter(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor
                              ) -> Optional[torch.Tensor]:
    """x[T, K/w] bf16 -> reduce_scatter(Q(x) dq(W)^T) [T/w, N] with the partial tiles pushed from the epilogue."""
    ws = _STATE["ws"]
    if ws is None:
        return None
    return ws.nvfp4_gemm_reduce_scatter(x, packed, scales, global_scale)


# ---------------------------------------------------------------------------------------------- fused or not, measured
# A fused kernel hides the transfer behind the GEMM but computes on the one-CTA GEMM (or carries copy CTAs); NCCL followed
# by the CTA-pair GEMM exposes the transfer but computes faster. Which one wins depends on the op, its shape and the
# number of ranks (at 2 ranks the transfer is small, at 8 it is as long as the GEMM), so every (op, shape) is timed once,
# at its first use, on the device, as the max over the ranks, and the faster variant is used from then on.
_CHOICE: Dict[tuple, bool] = {}
_AUTOTUNE = os.environ.get("HIPPO_FUSED_AUTOTUNE", "1") != "0"


def _trial_failed(ws, group) -> bool:
    """Collective: did a bounded device wait run out on any rank of ``group`` (status word set) since the last check? If
    so the status words are cleared and the arrival counters of the workspace reset, so that the run can go on with the
    NCCL + plain GEMM variant of the op that was being tried."""
    import torch.distributed as dist
    from ..ops import _ext
    dev = ws.mesh.device
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
    bad = torch.tensor([1.0 if _ext.device_status()[0] != 0 else 0.0], device=dev)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(bad, op=dist.ReduceOp.MAX, group=group)
    if float(bad) == 0.0:
        return False
    _ext.clear_device_status()
    ws.reset_counters()
    return True


def tuned(key: tuple, fused_fn: Callable[[], object], unfused_fn: Callable[[], object]):
    """Result of ``fused_fn()`` or ``unfused_fn()``, whichever was faster when ``key`` was first seen. Both compute the
    same values; every rank of the TP group must call this with the same key at the same point (the timing is collective).
    A ``fused_fn`` that returns None (shape not covered) settles the choice on the unfused path."""
    ws = _STATE["ws"]
    if ws is None:
        return unfused_fn()
    use = _CHOICE.get(key)
    if use is None and not _AUTOTUNE:
        use = True
    if use is not None:
        if use:
            out = fused_fn()
            if not _is_none(out):
                return out
        return unfused_fn()
    import torch.distributed as dist
    group = ws._group
    res, times = {}, {}
    for name, fn in (("unfused", unfused_fn), ("fused", fused_fn)):
        out = fn()                                            # warm-up (and the coverage check of the fused path)
        if _is_none(out):
            times[name] = float("inf")
            continue
        ts = []
        for _ in range(2):
            torch.cuda.synchronize()
            dist.barrier(group=group)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); out = fn(); e1.record(); e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor([min(ts)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        times[name], res[name] = float(t), out
    # the first use doubles as a probe: a fused kernel whose wait on a peer ran out on any rank is not used for this shape
    gave_up = times["fused"] != float("inf") and _trial_failed(ws, group)
    use = times["fused"] <= times["unfused"] and not gave_up
    _CHOICE[key] = use
    if ws.rank == 0:
        import logging
        logging.getLogger("hippo.r0").info(f"fused-comm choice {key}: fused {times['fused']:.3f} ms, "
                                           f"unfused {times['unfused']:.3f} ms -> {'fused' if use else 'unfused'}"
                                           + (" (a bounded wait ran out in the fused trial; counters reset)" if gave_up else ""))
    return res["fused" if use else "unfused"]


def _is_none(out) -> bool:
    return out is None or (isinstance(out, tuple) and out[0] is None)


def choices() -> Dict[tuple, bool]:
    return dict(_CHOICE)


def workspace():
    """The active symmetric workspace (None until setup())."""
    return _STATE["ws"]
