"""CUDA path of the vocab-parallel embedding (``csrc/embed.cu``): gather of the token shard's rows from the owning
ranks' weight mirrors over peer memory, and the pull-based weight gradient."""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from ._ext import lib, ptr, stream_ptr, check


def _ptr_arr(ptrs: Sequence[int]) -> C.Array:
    return (C.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def gather(ids: torch.Tensor, shard_ptrs: Sequence[int], Vl: int, D: int) -> torch.Tensor:
    """ids [n] int64 -> bf16 [n, D]; row of id v is read from shard v // Vl (device pointers of bf16 [Vl, D] arrays)."""
    ids = ids.to(torch.int64).contiguous()
    out = torch.empty((ids.numel(), D), dtype=torch.bfloat16, device=ids.device)
    check(lib().hippo_embed_gather(ptr(ids), _ptr_arr(shard_ptrs), len(shard_ptrs), Vl, D, ptr(out),
                                   C.c_longlong(ids.numel()), stream_ptr()), "embed_gather")
    return out


def grad(ids: torch.Tensor, grad_ptrs: Sequence[int], rows_per_rank: int, v0: int, Vl: int, D: int) -> torch.Tensor:
    """fp32 [Vl, D] gradient of the vocabulary rows [v0, v0 + Vl) from the bf16 output gradients of every token shard."""
    ids = ids.to(torch.int64).contiguous()
    dw = torch.zeros((Vl, D), dtype=torch.float32, device=ids.device)
    check(lib().hippo_embed_grad(ptr(ids), _ptr_arr(grad_ptrs), len(grad_ptrs), C.c_longlong(rows_per_rank),
                                 C.c_longlong(v0), Vl, D, ptr(dw), C.c_longlong(ids.numel()), stream_ptr()), "embed_grad")
    return dw
