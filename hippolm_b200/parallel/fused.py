"""Fused compute + collective kernels over NVSwitch peer memory (entry points).

``setup()`` allocates the symmetric workspace for the current TP group and switches the
sequence-parallel linears from "NCCL then GEMM" to the single-kernel paths in
``csrc/gemm_bf16.cu`` / ``csrc/gemm_fp4.cu`` / ``csrc/lce_fused.cu``. Until it is called (or on CPU) ``enabled()`` is False and the NCCL/gloo
baseline runs.
"""
from __future__ import annotations

from typing import Optional, Tuple

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


def workspace():
    """The active symmetric workspace (None until setup())."""
    return _STATE["ws"]
