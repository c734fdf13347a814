"""Python wrappers over the host C++ library (``csrc/host_fused.cpp``) with pure-torch fallbacks
(forced by ``HIPPO_FUSED_FORCE_PYLOOP=1``), mirroring ``param_offload/cpu_fused.py:913-1218``."""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Sequence

import torch

from ..ops import _ext


def _lib():
    if os.environ.get("HIPPO_FUSED_FORCE_PYLOOP") == "1":
        return None
    return _ext.host_lib()


def isa() -> str:
    """Which build of the host kernels this process uses: ``"avx512"`` or ``"avx2"`` (chosen once by CPUID;
    ``HIPPO_HOST_ISA=avx2`` forces the narrower one), ``"python"`` when the library is absent or bypassed."""
    lib = _lib()
    if lib is None:
        return "python"
    return "avx512" if lib.hippo_host_isa() == 1 else "avx2"


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise TypeError(f"host fused kernels take fp32/bf16, got {t.dtype}")


def _arrs(ts: Sequence[torch.Tensor]):
    n = len(ts)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in ts])
    numel = (C.c_int64 * n)(*[t.numel() for t in ts])
    dts = (C.c_int * n)(*[_dt(t) for t in ts])
    return ptrs, numel, dts, n


def fused_add_into_many(dsts: List[torch.Tensor], srcs: List[torch.Tensor]) -> None:
    lib = _lib()
    if lib is None or not dsts:
        for d, s in zip(dsts, srcs):
            d.add_(s.to(d.dtype))
        return
    dp, numel, ddt, n = _arrs(dsts)
    sp, _, sdt, _ = _arrs(srcs)
    lib.hippo_host_add_into_many(dp, sp, numel, ddt, sdt, n)


def fused_zero_many(ts: List[torch.Tensor]) -> None:
    lib = _lib()
    if lib is None or not ts:
        for t in ts:
            t.zero_()
        return
    n = len(ts)
    ptrs = (C.c_void_p * n)(*[t.data_ptr() for t in ts])
    nbytes = (C.c_int64 * n)(*[t.numel() * t.element_size() for t in ts])
    lib.hippo_host_zero_many(ptrs, nbytes, n)


def fused_scale_many(ts: List[torch.Tensor], scale: float) -> None:
    lib = _lib()
    if lib is None or not ts:
        for t in ts:
            t.mul_(scale)
        return
    p, numel, dt, n = _arrs(ts)
    lib.hippo_host_scale_many(p, numel, dt, n, C.c_float(scale))


def fused_l2_norm_sq(ts: List[torch.Tensor]) -> float:
    lib = _lib()
    if lib is None or not ts:
        return float(sum(t.double().pow(2).sum() for t in ts)) if ts else 0.0
    lib.hippo_host_l2_norm_sq.restype = C.c_double
    p, numel, dt, n = _arrs(ts)
    return float(lib.hippo_host_l2_norm_sq(p, numel, dt, n))


def fused_inf_nan_count(ts: List[torch.Tensor]) -> int:
    lib = _lib()
    if lib is None or not ts:
        return int(sum((~torch.isfinite(t.float())).sum() for t in ts)) if ts else 0
    lib.hippo_host_inf_nan_count.restype = C.c_int64
    p, numel, dt, n = _arrs(ts)
    return int(lib.hippo_host_inf_nan_count(p, numel, dt, n))


def fused_adam_step(grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor, b1: float, b2: float, eps: float,
                    step: int, grad_scale: float = 1.0, reference_compat: bool = False) -> None:
    """Updates m, v in place and overwrites ``grad`` with the update factor."""
    lib = _lib()
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    if lib is None:
        g = grad.float() * grad_scale
        mf = m.float().mul_(b1).add_(g, alpha=1 - b1)
        vf = v.float().mul_(b2).add_((mf * mf if reference_compat else g * g), alpha=1 - b2)
        m.copy_(mf); v.copy_(vf)
        upd = mf / ((vf / bc2).sqrt() + eps) if reference_compat else (mf / bc1) / ((vf / bc2).sqrt() + eps)
        grad.copy_(upd)
        return
    lib.hippo_host_adam_step(C.c_void_p(grad.data_ptr()), C.c_void_p(m.data_ptr()), C.c_void_p(v.data_ptr()),
                             C.c_int64(grad.numel()), _dt(grad), _dt(m), _dt(v), C.c_float(b1), C.c_float(b2),
                             C.c_float(eps), C.c_float(bc1), C.c_float(bc2), C.c_float(grad_scale),
                             int(reference_compat))
