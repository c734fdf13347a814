"""CUDA execution path: autograd Functions over the sm_100a kernels in ``hippolm_b200/csrc``."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch

from . import _ext
from ._ext import lib, ptr, stream_ptr, check

_c = ctypes


# ----------------------------------------------------------------------------- GEMM
def _gemm(a: torch.Tensor, b: torch.Tensor, layout: int, M: int, N: int, K: int,
          out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, accumulate: bool = False,
          alpha: float = 1.0, max_ctas: int = 0) -> torch.Tensor:
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "bf16 GEMM operands required"
    if a.stride(-1) != 1 or (a.stride(0) % 8) or (a.data_ptr() % 16):
        a = a.contiguous()
    if b.stride(-1) != 1 or (b.stride(0) % 8) or (b.data_ptr() % 16):
        b = b.contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    rc = lib().hippo_gemm_bf16(ptr(a), ptr(b), ptr(out), M, N, K, _c.c_longlong(a.stride(0)),
                               _c.c_longlong(b.stride(0)), _c.c_longlong(out.stride(0)), layout,
                               1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
                               _c.c_float(alpha), max_ctas, stream_ptr())
    check(rc, "hippo_gemm_bf16")
    return out


def _pad_cols(x: torch.Tensor, mult: int = 8) -> torch.Tensor:
    n = x.shape[1]
    if n % mult == 0:
        return x
    return torch.nn.functional.pad(x, (0, mult - n % mult))


def gemm_nt(a, b, out_dtype=None):
    """a[M,K] @ b[N,K]^T"""
    M, K = a.shape
    N = b.shape[0]
    od = out_dtype or a.dtype
    a, b = a.to(torch.bfloat16), b.to(torch.bfloat16)
    if K % 8:
        a, b = _pad_cols(a), _pad_cols(b)
    if N % 8:
        y = _gemm(a, b, 0, M, N, a.shape[1], out=torch.empty((M, (N + 7) // 8 * 8), dtype=torch.bfloat16,
                                                             device=a.device)[:, :N])
        return y.contiguous().to(od)
    return _gemm(a, b, 0, M, N, a.shape[1], out_dtype=torch.float32 if od == torch.float32 else torch.bfloat16).to(od)


def gemm_nn(a, b, out_dtype=None):
    """a[M,N] @ b[N,K] -> [M,K]   (contraction over a's columns / b's rows)"""
    M, Nc = a.shape
    K = b.shape[1]
    od = out_dtype or a.dtype
    a, b = a.to(torch.bfloat16), b.to(torch.bfloat16)
    if Nc % 8 or K % 8:
        return gemm_nt(a, b.t().contiguous(), od)
    return _gemm(a, b, 1, M, K, Nc, out_dtype=torch.float32 if od == torch.float32 else torch.bfloat16).to(od)


def gemm_tn(a, b, out_dtype=None):
    """a[M,N]^T @ b[M,K] -> [N,K]   (contraction over rows)"""
    Mc, N = a.shape
    K = b.shape[1]
    od = out_dtype or a.dtype
    a, b = a.to(torch.bfloat16), b.to(torch.bfloat16)
    if N % 8 or K % 8:
        return gemm_nt(a.t().contiguous(), b.t().contiguous(), od)
    return _gemm(a, b, 2, N, K, Mc, out_dtype=torch.float32 if od == torch.float32 else torch.bfloat16).to(od)
