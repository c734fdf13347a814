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
    def forward(ctx, q, k, v, g, beta, h0, cu_seqlens, skip_saved=False):
        """``skip_saved``: keep only the inputs and the two per-chunk state tensors for backward and recompute the
        per-chunk WY / A-matrix tensors there with one extra launch of the intra-chunk kernel (the reference's
        ``kda_skip_aqk_akk_saved`` drops Aqk and Akk, ``fla/ops/kda/chunk.py:91-106``; here G, w, qg, kg, Aqk, Ainv
        and Akk all go: 11 KB -> 3 KB of saved activations per token-head at head_dim 128)."""
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
        ctx.skip_saved = bool(skip_saved)
        if ctx.skip_saved:
            ctx.save_for_backward(q, k, v, beta, g, vnew, Sst, cs, cl, sc, so)
        else:
            ctx.save_for_backward(q, k, v, beta, G, w, qg, kg, Aqk, Ainv, Akk, vnew, Sst, cs, cl, sc, so)
        ctx.dims = (T, H, DK, NC, N)
        ctx.has_h0 = h0 is not None
        return o, fin

    @staticmethod
    def backward(ctx, do, dfin):
        from . import kda_bwd_cuda
        return kda_bwd_cuda.backward(ctx, do, dfin)


def recompute_intra(q, k, v, g, beta, cs, cl, NC, H, DK):
    """(G, w, qg, kg, Aqk, Ainv, Akk) of the forward pass, rebuilt from the inputs."""
    dev = q.device
    bf = dict(dtype=torch.bfloat16, device=dev)
    G = torch.empty((NC, H, 64, DK), dtype=torch.float32, device=dev)
    w, u, qg, kg = (torch.empty((NC, H, 64, DK), **bf) for _ in range(4))
    Aqk, Ainv, Akk = (torch.empty((NC, H, 64, 64), **bf) for _ in range(3))
    check(lib().hippo_kda_fwd_intra(ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(cs), ptr(cl), NC, H, DK, ptr(G), ptr(w),
                                    ptr(u), ptr(qg), ptr(kg), ptr(Aqk), ptr(Ainv), ptr(Akk), stream_ptr()), "kda_fwd_intra")
    return G, w, qg, kg, Aqk, Ainv, Akk


def kda_recurrent_fwd(q, k, v, g, beta, h0, cu_seqlens):
    """Token-recurrent forward (``csrc/kda_recurrent.cu``): (o [T,H,V] bf16, final state [N,H,K,V] fp32). No backward."""
    T, H, DK = q.shape
    assert v.shape[-1] == DK and DK in (64, 128), "CUDA KDA supports K == V in {64, 128}"
    q, k, v = (t.detach().to(torch.bfloat16).contiguous() for t in (q, k, v))
    g, beta = g.detach().float().contiguous(), beta.detach().float().contiguous()
    cu = cu_seqlens.to(torch.int32).contiguous()
    N = cu.numel() - 1
    o = torch.empty((T, H, DK), dtype=torch.bfloat16, device=q.device)
    fin = torch.empty((N, H, DK, DK), dtype=torch.float32, device=q.device)
    h0c = h0.detach().float().contiguous() if h0 is not None else None
    check(lib().hippo_kda_recurrent_fwd(ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(cu), N, H, DK, ptr(h0c), ptr(o),
                                        ptr(fin), stream_ptr()), "kda_recurrent_fwd")
    return o, fin


def kda(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_qk_l2norm, skip_saved: bool = False,
        mode: str = "chunk"):
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
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad
                                                 for t in (q, k, v, g, beta, initial_state))
    if mode == "fused_recurrent" and not needs_grad:
        # inference / decode: the token recurrence in one kernel; training in this mode uses the chunk kernels, whose
        # result is the same function (the recurrent form has no backward, as in fla/ops/kda/fused_recurrent.py)
        return kda_recurrent_fwd(q, k, v, g, beta, initial_state, cu_seqlens)
    return _KDAFunction.apply(q, k, v, g, beta, initial_state, cu_seqlens, skip_saved)
