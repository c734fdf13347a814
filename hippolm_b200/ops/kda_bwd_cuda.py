"""Backward of the CUDA KDA op: four kernels in ``csrc/kda_bwd.cu`` (reverse state recurrence, then
three per-chunk kernels)."""
from __future__ import annotations

import torch

from ._ext import lib, ptr, stream_ptr, check


def backward(ctx, do, dfin):
    T, H, DK, NC, N = ctx.dims
    if getattr(ctx, "skip_saved", False):
        from .kda_cuda import recompute_intra
        q, k, v, beta, g, vnew, Sst, cs, cl, sc, so = ctx.saved_tensors
        G, w, qg, kg, Aqk, Ainv, Akk = recompute_intra(q, k, v, g, beta, cs, cl, NC, H, DK)
    else:
        q, k, v, beta, G, w, qg, kg, Aqk, Ainv, Akk, vnew, Sst, cs, cl, sc, so = ctx.saved_tensors
    dev = q.device
    do = do.to(torch.bfloat16).contiguous()
    dfin_c = dfin.float().contiguous() if dfin is not None else None
    bf = dict(dtype=torch.bfloat16, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    dvn, dw, dbk = (torch.empty((NC, H, 64, DK), **bf) for _ in range(3))
    dSst = torch.empty((NC, H, DK, DK), **bf)
    dAqk, dKK = torch.empty((NC, H, 64, 64), **bf), torch.empty((NC, H, 64, 64), **bf)
    dq_acc, dk_acc, dG_acc = (torch.empty((NC, H, 64, DK), **f32) for _ in range(3))
    # dq / dk leave the last kernel as bf16 (the dtype of q / k): no cast between it and the consumer
    dq, dk = (torch.empty((T, H, DK), **bf) for _ in range(2))
    dg = torch.empty((T, H, DK), **f32)
    dv = torch.empty((T, H, DK), **bf)
    dbeta = torch.empty((T, H), **f32)
    dh0 = torch.empty((N, H, DK, DK), **f32) if ctx.has_h0 else None
    check(lib().hippo_kda_bwd(ptr(q), ptr(k), ptr(v), ptr(beta), ptr(G), ptr(w), ptr(qg), ptr(kg), ptr(Aqk), ptr(Ainv),
                              ptr(Akk), ptr(vnew), ptr(Sst), ptr(do), ptr(dfin_c), ptr(cs), ptr(cl), ptr(sc), ptr(so), NC, N, H,
                              DK, ptr(dvn), ptr(dSst), ptr(dw), ptr(dAqk), ptr(dKK), ptr(dbk), ptr(dq_acc), ptr(dk_acc),
                              ptr(dG_acc), ptr(dq), ptr(dk), ptr(dv), ptr(dg), ptr(dbeta), ptr(dh0), stream_ptr()),
          "kda_bwd")
    return dq, dk, dv, dg, dbeta, dh0, None, None
