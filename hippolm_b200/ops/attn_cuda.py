"""CUDA path of causal varlen attention: tcgen05 kernels for head_dim 128 (``csrc/attention_tc.cu``), mma.sync kernels
for head_dim 64 (``csrc/attention.cu``). The reference has no softmax-attention layer."""
from __future__ import annotations

import ctypes as _c
import os

import torch

from ._ext import lib, ptr, stream_ptr, check

_CACHE = {"key": None}
_CACHE128 = {"key": None}
_USE_TC = os.environ.get("HIPPO_ATTN_TC", "1") != "0"           # tcgen05 forward (head_dim 128)
_USE_TC_BWD = os.environ.get("HIPPO_ATTN_TC_BWD", "1") != "0"   # tcgen05 backward (needs the tcgen05 forward's tiles)


def tile_tables_128(cu_seqlens: torch.Tensor, T: int):
    """128-row query tiles (start, length, document start) for the tcgen05 forward kernel."""
    key = (cu_seqlens.data_ptr(), cu_seqlens._version, cu_seqlens.numel(), T)
    if _CACHE128["key"] == key and _CACHE128.get("ref") is cu_seqlens:
        return _CACHE128["val"]
    N = cu_seqlens.numel() - 1
    cu = cu_seqlens.to(torch.int32).contiguous()
    nt = (T + 127) // 128 + N
    ts, tl, t0, te = (torch.empty(nt, dtype=torch.int32, device=cu.device) for _ in range(4))
    check(lib().hippo_attn_build_tiles_rows(ptr(cu), N, 128, ptr(ts), ptr(tl), ptr(t0), ptr(te), nt, stream_ptr()),
          "attn_build_tiles_rows")
    val = (ts, tl, t0, te, nt)
    _CACHE128.update(key=key, val=val, ref=cu_seqlens)
    return val


def tile_tables(cu_seqlens: torch.Tensor, T: int):
    key = (cu_seqlens.data_ptr(), cu_seqlens._version, cu_seqlens.numel(), T)
    if _CACHE["key"] == key and _CACHE.get("ref") is cu_seqlens:
        return _CACHE["val"]
    N = cu_seqlens.numel() - 1
    cu = cu_seqlens.to(torch.int32).contiguous()
    nt = (T + 63) // 64 + N
    ts, tl, t0, te = (torch.empty(nt, dtype=torch.int32, device=cu.device) for _ in range(4))
    check(lib().hippo_attn_build_tiles(ptr(cu), N, ptr(ts), ptr(tl), ptr(t0), ptr(te), nt, stream_ptr()),
          "attn_build_tiles")
    val = (ts, tl, t0, te, nt)
    _CACHE.update(key=key, val=val, ref=cu_seqlens)
    return val


class _Attn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, scale):
        T, H, DH = q.shape
        assert DH in (64, 128), "CUDA attention supports head_dim 64 or 128"
        q, k, v = (t.to(torch.bfloat16).contiguous() for t in (q, k, v))
        use_tc = DH == 128 and _USE_TC
        if not use_tc:
            ts, tl, t0, te, nt = tile_tables(cu_seqlens, T)
        o = torch.empty_like(q)
        lse = torch.empty((T, H), dtype=torch.float32, device=q.device)
        if use_tc:
            # tcgen05 forward: S and P V in TMEM, 128 x 128 tiles fed by TMA
            ts8, tl8, t08, te8, nt8 = tile_tables_128(cu_seqlens, T)
            check(lib().hippo_attn_fwd_tc(ptr(q), ptr(k), ptr(v), ptr(ts8), ptr(tl8), ptr(t08), nt8, H, _c.c_longlong(T),
                                          _c.c_float(scale), ptr(o), ptr(lse), stream_ptr()), "attn_fwd_tc")
            ts, tl, t0, te, nt = ts8, tl8, t08, te8, nt8            # the backward kernels use the same 128-row tiles
        else:
            check(lib().hippo_attn_fwd(ptr(q), ptr(k), ptr(v), ptr(ts), ptr(tl), ptr(t0), nt, H, DH, _c.c_float(scale),
                                       ptr(o), ptr(lse), stream_ptr()), "attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse, ts, tl, t0, te)
        ctx.meta = (T, H, DH, nt, scale)
        ctx.tc = bool(use_tc)
        ctx.cu = cu_seqlens
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, ts, tl, t0, te = ctx.saved_tensors
        T, H, DH, nt, scale = ctx.meta
        do = do.to(torch.bfloat16).contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty((T, H), dtype=torch.float32, device=q.device)
        if ctx.tc and _USE_TC_BWD:
            check(lib().hippo_attn_bwd_tc(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(delta), ptr(ts), ptr(tl),
                                          ptr(t0), ptr(te), nt, H, _c.c_longlong(T), _c.c_float(scale), ptr(dq), ptr(dk),
                                          ptr(dv), stream_ptr()), "attn_bwd_tc")
            return dq, dk, dv, None, None
        if ctx.tc:
            ts, tl, t0, te, nt = tile_tables(ctx.cu, T)
        check(lib().hippo_attn_bwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(delta), ptr(ts), ptr(tl),
                                   ptr(t0), ptr(te), nt, H, DH, _c.c_longlong(T), _c.c_float(scale), ptr(dq), ptr(dk),
                                   ptr(dv), stream_ptr()), "attn_bwd")
        return dq, dk, dv, None, None


def causal_attention(q, k, v, cu_seqlens, scale):
    T, H, DH = q.shape
    if scale is None:
        scale = DH ** -0.5
    if cu_seqlens is None:
        cu_seqlens = torch.tensor([0, T], dtype=torch.int32, device=q.device)
    return _Attn.apply(q, k, v, cu_seqlens, float(scale))
