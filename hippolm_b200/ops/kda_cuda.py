"""CUDA path of Kimi delta attention: chunked forward / backward kernels (``csrc/kda_fwd.cu``,
``csrc/kda_bwd.cu``). Inputs are token-major packed streams; see :mod:`hippolm_b200.ref.kda`."""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch

from ._ext import lib, ptr, stream_ptr, check

_TABLE_CACHE = {"key": None, "val": None}


def chunk_tables(cu_seqlens: torch.Tensor, T: int):
    """(chunk_start, chunk_len, seq_chunk, nc_max, N) built on the device without a host sync."""
    key = (cu_seqlens.data_ptr(), cu_seqlens._version, cu_seqlens.numel(), T)
    if _TABLE_CACHE["key"] == key and _TABLE_CACHE["ref"] is cu_seqlens:
        return _TABLE_CACHE["val"]
    N = cu_seqlens.numel() - 1
    cu = cu_seqlens.to(torch.int32).contiguous()
    nc_max = (T + 63) // 64 + N
    cs = torch.empty(nc_max, dtype=torch.int32, device=cu.device)
    cl = torch.empty(nc_max, dtype=torch.int32, device=cu.device)
    sc = torch.empty(N + 1, dtype=torch.int32, device=cu.device)
    so = torch.empty(N, dtype=torch.int32, device=cu.device)
    check(lib().hippo_kda_build_chunks(ptr(cu), N, ptr(cs), ptr(cl), ptr(sc), ptr(so), nc_max, stream_ptr()),
          "kda_build_chunks")
    val = (cs, cl, sc, so, nc_max, N)
    _TABLE_CACHE.update(key=key, val=val, ref=cu_seqlens)
    return val


class _KDAFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, h0, cu_seqlens):
        T, H, DK = q.shape
        assert v.shape[-1] == DK and DK in (64, 128), "CUDA KDA supports K == V in {64, 128}"
        dev = q.device
        q, k, v = (t.to(torch.bfloat16).contiguous() for t in (q, k, v))
        g, beta = g.float().contiguous(), beta.float().contiguous()
        cs, cl, sc, so, NC, N = chunk_tables(cu_seqlens, T)
        bf = dict(dtype=torch.bfloat16, device=dev)
        G = torch.empty((NC, H, 64, DK), dtype=torch.float32, device=dev)
        w, u, qg, kg, vnew = (torch.empty((NC, H, 64, DK), **bf) for _ in range(5))
        Aqk, Ainv, Akk = (torch.empty((NC, H, 64, 64), **bf) for _ in range(3))
        Sst = torch.empty((NC, H, DK, DK), **bf)
        o = torch.empty((T, H, DK), **bf)
        fin = torch.empty((N, H, DK, DK), dtype=torch.float32, device=dev)
        h0c = h0.float().contiguous() if h0 is not None else None
        check(lib().hippo_kda_fwd(ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(cs), ptr(cl), ptr(sc), ptr(so), NC, N, H, DK,
                                  ptr(h0c), ptr(G), ptr(w), ptr(u), ptr(qg), ptr(kg), ptr(Aqk), ptr(Ainv), ptr(Akk), ptr(vnew),
                                  ptr(Sst), ptr(o), ptr(fin), stream_ptr()), "kda_fwd")
        ctx.save_for_backward(q, k, v, beta, G, w, qg, kg, Aqk, Ainv, Akk, vnew, Sst, cs, cl, sc, so)
        ctx.dims = (T, H, DK, NC, N)
        ctx.has_h0 = h0 is not None
        return o, fin

    @staticmethod
    def backward(ctx, do, dfin):
        from . import kda_bwd_cuda
        return kda_bwd_cuda.backward(ctx, do, dfin)


def kda(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_qk_l2norm):
    T, H, K = q.shape
    if scale is None:
        scale = K ** -0.5
    if cu_seqlens is None:
        cu_seqlens = torch.tensor([0, T], dtype=torch.int32, device=q.device)
    if use_qk_l2norm:
        from ..ref.kda import l2norm
        q, k = l2norm(q.float()), l2norm(k.float())
    if scale != 1.0:
        q = q.float() * scale
    return _KDAFunction.apply(q, k, v, g, beta, initial_state, cu_seqlens)
