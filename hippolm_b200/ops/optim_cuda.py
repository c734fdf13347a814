"""CUDA path of the optimizer update kernels (``csrc/misc_ops.cu``)."""
from __future__ import annotations

import ctypes as _c

import torch

from ._ext import lib, ptr, stream_ptr, check


def _isbf(t):
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise TypeError(f"unsupported dtype {t.dtype}")


def adamw_update(p, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    assert p.is_contiguous() and m.is_contiguous() and v.is_contiguous()
    g = g.contiguous()
    if all(t.dtype == torch.bfloat16 for t in (p, g, m, v)) and p.numel() % 8 == 0:
        check(lib().hippo_adamw_bf16(ptr(p), ptr(g), ptr(m), ptr(v), _c.c_longlong(p.numel()), _c.c_float(lr),
                                     _c.c_float(beta1), _c.c_float(beta2), _c.c_float(eps), _c.c_float(wd),
                                     _c.c_float(1 - beta1 ** step), _c.c_float(1 - beta2 ** step),
                                     _c.c_float(grad_scale), stream_ptr()), "adamw_bf16")
        return
    check(lib().hippo_adamw(ptr(p), ptr(g), ptr(m), ptr(v), _c.c_longlong(p.numel()), _isbf(p), _isbf(g), _isbf(m),
                            _isbf(v), _c.c_float(lr), _c.c_float(beta1), _c.c_float(beta2), _c.c_float(eps),
                            _c.c_float(wd), _c.c_float(1 - beta1 ** step), _c.c_float(1 - beta2 ** step),
                            _c.c_float(grad_scale), stream_ptr()), "adamw")


def sumsq_into(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[0] += sum(x^2) (fp32 accumulate)."""
    x = x.contiguous()
    check(lib().hippo_sumsq(ptr(x), _c.c_longlong(x.numel()), _isbf(x), ptr(out), stream_ptr()), "sumsq")


def sumsq_multi(items, out: torch.Tensor) -> None:
    """items: [(tensor, slot)]; out[slot] += sum(tensor^2) for all of them in ONE launch (table of pointers uploaded
    from a small pinned buffer). Tensors must be contiguous bf16 / fp32."""
    import struct
    items = [(t, sl) for t, sl in items if t.numel() > 0]
    if not items:
        return
    rec, piece = [], 0
    for t, slot in items:
        assert t.is_contiguous()
        rec.append(struct.pack("<QqiiQ", t.data_ptr(), t.numel(), _isbf(t), slot, piece))
        piece += (t.numel() + 2047) // 2048
    raw = b"".join(rec)
    host = torch.frombuffer(bytearray(raw), dtype=torch.uint8).pin_memory()
    tab = host.to(out.device, non_blocking=True)
    check(lib().hippo_sumsq_multi(ptr(tab), len(items), _c.c_longlong(piece), ptr(out), stream_ptr()), "sumsq_multi")
    tab.record_stream(torch.cuda.current_stream())
