"""CUDA path of the block attention residual mix (``csrc/misc_ops.cu``)."""
from __future__ import annotations

import ctypes as _c

import torch

from ._ext import lib, ptr, stream_ptr, check


def _ptr_array(ts):
    arr = (_c.c_void_p * len(ts))()
    for i, t in enumerate(ts):
        arr[i] = t.data_ptr()
    return arr


class _AttnRes(torch.autograd.Function):
    @staticmethod
    def forward(ctx, query, norm_weight, eps, *sources):
        N = len(sources)
        T, D = sources[0].shape
        H = query.shape[0]
        srcs = [s.to(torch.bfloat16).contiguous() for s in sources]
        qb, wb = query.to(torch.bfloat16).contiguous(), norm_weight.to(torch.bfloat16).contiguous()
        out = torch.empty((T, D), dtype=torch.bfloat16, device=srcs[0].device)
        alpha = torch.empty((N, T, H), dtype=torch.float32, device=out.device)
        rstd = torch.empty((N, T), dtype=torch.float32, device=out.device)
        check(lib().hippo_attnres_fwd(_ptr_array(srcs), N, ptr(qb), ptr(wb), ptr(out), ptr(alpha), ptr(rstd),
                                      _c.c_longlong(T), D, H, _c.c_float(eps), stream_ptr()), "attnres_fwd")
        ctx.save_for_backward(qb, wb, out, alpha, rstd, *srcs)
        ctx.meta = (N, T, D, H, query.dtype, norm_weight.dtype, [s.dtype for s in sources])
        return out.to(sources[0].dtype)

    @staticmethod
    def backward(ctx, dout):
        qb, wb, out, alpha, rstd, *srcs = ctx.saved_tensors
        N, T, D, H, qdt, wdt, sdts = ctx.meta
        dout = dout.to(torch.bfloat16).contiguous()
        dsrcs = [torch.empty_like(s) for s in srcs]
        dq = torch.zeros(D, dtype=torch.float32, device=out.device)
        dw = torch.zeros(D, dtype=torch.float32, device=out.device)
        check(lib().hippo_attnres_bwd(_ptr_array(srcs), N, ptr(qb), ptr(wb), ptr(out), ptr(dout), ptr(alpha), ptr(rstd),
                                      _ptr_array(dsrcs), ptr(dq), ptr(dw), _c.c_longlong(T), D, H, stream_ptr()),
              "attnres_bwd")
        return (dq.view(H, D // H).to(qdt), dw.to(wdt), None) + tuple(d.to(dt) for d, dt in zip(dsrcs, sdts))


def attn_res(sources, query, norm_weight, eps):
    return _AttnRes.apply(query, norm_weight, float(eps), *sources)
