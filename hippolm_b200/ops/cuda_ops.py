"""CUDA execution path: autograd Functions over the sm_100a kernels in ``hippolm_b200/csrc``."""
from __future__ import annotations

import os
import ctypes
from typing import List, Optional, Tuple

import torch

from . import _ext
from ._ext import lib, ptr, stream_ptr, check

_c = ctypes


# ----------------------------------------------------------------------------- GEMM
def _gemm(a: torch.Tensor, b: torch.Tensor, layout: int, M: int, N: int, K: int,
          out: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16, accumulate: bool = False,
          alpha: float = 1.0, max_ctas: int = 0, kernel: str = "auto") -> torch.Tensor:
    """kernel: "auto" (CTA-pair kernel for M > 128, else one-CTA), "1sm" or "2sm" (explicit, for tests / benches)."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "bf16 GEMM operands required"
    if a.stride(-1) != 1 or (a.stride(0) % 8) or (a.data_ptr() % 16):
        a = a.contiguous()
    if b.stride(-1) != 1 or (b.stride(0) % 8) or (b.data_ptr() % 16):
        b = b.contiguous()
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if kernel == "2sm":
        rc = lib().hippo_gemm_bf16_2sm(ptr(a), ptr(b), ptr(out), None, M, N, K, _c.c_longlong(a.stride(0)),
                                       _c.c_longlong(b.stride(0)), _c.c_longlong(out.stride(0)), _c.c_longlong(0),
                                       layout, 1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
                                       _c.c_float(alpha), _c.c_float(0.0), stream_ptr())
        check(rc, "hippo_gemm_bf16_2sm")
        return out
    ks = _splitk_factor(M, N, K) if kernel == "auto" else 1
    if ks > 1:
        # too few 256x256 output tiles for 74 CTA pairs (weight gradients of narrow projections): cut the contraction
        ws = torch.empty(ks * M * N, dtype=torch.float32, device=a.device)
        rc = lib().hippo_gemm_bf16_splitk(ptr(a), ptr(b), ptr(out), ptr(ws), M, N, K, _c.c_longlong(a.stride(0)),
                                          _c.c_longlong(b.stride(0)), _c.c_longlong(out.stride(0)), layout,
                                          1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
                                          _c.c_float(alpha), ks, stream_ptr())
        check(rc, "hippo_gemm_bf16_splitk")
        return out
    fn = lib().hippo_gemm_bf16_1sm if kernel == "1sm" else lib().hippo_gemm_bf16
    rc = fn(ptr(a), ptr(b), ptr(out), M, N, K, _c.c_longlong(a.stride(0)),
                               _c.c_longlong(b.stride(0)), _c.c_longlong(out.stride(0)), layout,
                               1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
                               _c.c_float(alpha), max_ctas, stream_ptr())
    check(rc, "hippo_gemm_bf16")
    return out


_SPLITK = os.environ.get("HIPPO_GEMM_SPLITK", "1") != "0"


def _splitk_factor(M: int, N: int, K: int, clusters: int = 74) -> int:
    """Number of K slices for the CTA-pair kernel: the factor that minimises (waves of 256x256 work items) / slices plus
    the cost of the reduction pass. 1 = plain launch. Only long contractions with few output tiles qualify."""
    if not _SPLITK or M <= 128 or N % 4 or K < 4096:
        return 1
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    if tiles >= 2 * clusters:
        return 1
    best, best_cost = 1, float(-(-tiles // clusters))
    for s in (2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64):
        if K < 2048 * s or tiles * s > 8 * clusters or s * M * N * 4 > (1 << 28):
            break
        cost = (-(-tiles * s // clusters)) / s + 0.03 + (s + 1) * 467.0 / K
        if cost < 0.9 * best_cost:
            best, best_cost = s, cost
    return best


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


# ----------------------------------------------------------------------------- row ops
def _bf(x):
    return x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        xs = x.shape
        D = xs[-1]
        x2 = _bf(x).reshape(-1, D).contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        check(lib().hippo_rmsnorm_fwd(ptr(x2), ptr(_bf(w)), ptr(y), ptr(rstd), _c.c_longlong(T), D,
                                      _c.c_float(eps), stream_ptr()), "rmsnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.xs, ctx.xdtype = xs, x.dtype
        return y.view(xs).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        T, D = x2.shape
        dy2 = _bf(dy).reshape(T, D).contiguous()
        dx = torch.empty_like(x2)
        nb = min(T, 148 * 4)
        part = torch.empty((nb, D), dtype=torch.float32, device=x2.device)
        dw = torch.empty(D, dtype=torch.float32, device=x2.device)
        check(lib().hippo_rmsnorm_bwd(ptr(x2), ptr(_bf(w)), ptr(dy2), ptr(rstd), ptr(dx), ptr(part), ptr(dw),
                                      _c.c_longlong(T), D, nb, stream_ptr()), "rmsnorm_bwd")
        return dx.view(ctx.xs).to(ctx.xdtype), dw.to(w.dtype), None


def rmsnorm(x, w, eps):
    return _RMSNorm.apply(x, w, eps)


class _AddRMSNorm(torch.autograd.Function):
    """(x + res, rmsnorm(x + res) * w) in one kernel; backward folds the gradient of the sum that arrives through the
    residual path into the norm's backward kernel and hands the same tensor to both addends."""

    @staticmethod
    def forward(ctx, x, res, w, eps):
        xs = x.shape
        D = xs[-1]
        x2, r2 = _bf(x).reshape(-1, D).contiguous(), _bf(res).reshape(-1, D).contiguous()
        T = x2.shape[0]
        ssum, y = torch.empty_like(x2), torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        check(lib().hippo_add_rmsnorm_fwd(ptr(x2), ptr(r2), ptr(_bf(w)), ptr(ssum), ptr(y), ptr(rstd), _c.c_longlong(T), D,
                                          _c.c_float(eps), stream_ptr()), "add_rmsnorm_fwd")
        ctx.save_for_backward(ssum, w, rstd)
        ctx.xs, ctx.xdtype = xs, x.dtype
        return ssum.view(xs).to(x.dtype), y.view(xs).to(x.dtype)

    @staticmethod
    def backward(ctx, dsum, dy):
        ssum, w, rstd = ctx.saved_tensors
        T, D = ssum.shape
        if dy is None:
            return dsum, dsum, None, None
        dy2 = _bf(dy).reshape(T, D).contiguous()
        dres = _bf(dsum).reshape(T, D).contiguous() if dsum is not None else None
        dx = torch.empty_like(ssum)
        nb = min(T, 148 * 4)
        part = torch.empty((nb, D), dtype=torch.float32, device=ssum.device)
        dw = torch.empty(D, dtype=torch.float32, device=ssum.device)
        check(lib().hippo_rmsnorm_bwd_res(ptr(ssum), ptr(_bf(w)), ptr(dy2), ptr(dres), ptr(rstd), ptr(dx), ptr(part), ptr(dw),
                                          _c.c_longlong(T), D, nb, stream_ptr()), "rmsnorm_bwd_res")
        d = dx.view(ctx.xs).to(ctx.xdtype)
        return d, d, dw.to(w.dtype), None


def add_rmsnorm(x, res, w, eps):
    return _AddRMSNorm.apply(x, res, w, eps)


class _GatedRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, o, gate, w, eps):
        V = o.shape[-1]
        o2, g2 = _bf(o).contiguous(), _bf(gate).contiguous()
        rows = o2.numel() // V
        y = torch.empty_like(o2)
        rstd = torch.empty(rows, dtype=torch.float32, device=o.device)
        check(lib().hippo_gated_rmsnorm_fwd(ptr(o2), ptr(g2), ptr(_bf(w)), ptr(y), ptr(rstd), _c.c_longlong(rows), V,
                                            _c.c_float(eps), stream_ptr()), "gated_rmsnorm_fwd")
        ctx.save_for_backward(o2, g2, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        o2, g2, w, rstd = ctx.saved_tensors
        V = o2.shape[-1]
        rows = o2.numel() // V
        dy2 = _bf(dy).contiguous()
        do, dg = torch.empty_like(o2), torch.empty_like(g2)
        dw = torch.zeros(V, dtype=torch.float32, device=o2.device)
        check(lib().hippo_gated_rmsnorm_bwd(ptr(o2), ptr(g2), ptr(_bf(w)), ptr(dy2), ptr(rstd), ptr(do), ptr(dg),
                                            ptr(dw), _c.c_longlong(rows), V, stream_ptr()), "gated_rmsnorm_bwd")
        return do, dg, dw.to(w.dtype), None


def gated_rmsnorm(o, gate, w, eps):
    return _GatedRMSNorm.apply(o, gate, w, eps)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        gu = _bf(gu).contiguous()
        T, I2 = gu.shape
        a = torch.empty((T, I2 // 2), dtype=torch.bfloat16, device=gu.device)
        check(lib().hippo_swiglu_fwd(ptr(gu), ptr(a), _c.c_longlong(T), I2 // 2, stream_ptr()), "swiglu_fwd")
        ctx.save_for_backward(gu)
        return a

    @staticmethod
    def backward(ctx, da):
        (gu,) = ctx.saved_tensors
        T, I2 = gu.shape
        dgu = torch.empty_like(gu)
        check(lib().hippo_swiglu_bwd(ptr(gu), ptr(_bf(da).contiguous()), ptr(dgu), _c.c_longlong(T), I2 // 2,
                                     stream_ptr()), "swiglu_bwd")
        return dgu


def swiglu(gu):
    return _SwiGLU.apply(gu)


class _Silu(torch.autograd.Function):
    """SiLU through the row-op kernel (forward); the backward is elementwise torch on the saved input."""

    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        y = torch.empty_like(x)
        check(lib().hippo_silu_fwd(ptr(x), ptr(y), _c.c_longlong(x.numel()), stream_ptr()), "silu_fwd")
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        xf = x.float()
        sg = torch.sigmoid(xf)
        return (dy.float() * sg * (1 + xf * (1 - sg))).to(dy.dtype)


def silu(x):
    if x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0:
        return _Silu.apply(x)
    return torch.nn.functional.silu(x)


class _KDAGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, A, b, safe, lower):
        T, H, K = x.shape
        x2 = _bf(x).contiguous()
        g = torch.empty((T, H, K), dtype=torch.float32, device=x.device)
        Af = A.float().contiguous()
        bf_ = b.float().contiguous() if b is not None else None
        check(lib().hippo_kda_gate_fwd(ptr(x2), ptr(Af), ptr(bf_), ptr(g), _c.c_longlong(T), H, K, int(safe),
                                       _c.c_float(lower), stream_ptr()), "kda_gate_fwd")
        ctx.save_for_backward(x2, Af, bf_ if bf_ is not None else Af)
        ctx.has_b, ctx.safe, ctx.lower = b is not None, safe, lower
        ctx.dts = (x.dtype, A.dtype, b.dtype if b is not None else None)
        return g

    @staticmethod
    def backward(ctx, dg):
        x2, Af, bf_ = ctx.saved_tensors
        T, H, K = x2.shape
        dg = dg.float().contiguous()
        dx = torch.empty_like(x2)
        dA = torch.zeros(H, dtype=torch.float32, device=x2.device)
        db = torch.zeros(H * K, dtype=torch.float32, device=x2.device) if ctx.has_b else None
        check(lib().hippo_kda_gate_bwd(ptr(x2), ptr(Af), ptr(bf_ if ctx.has_b else None), ptr(dg), ptr(dx), ptr(dA),
                                       ptr(db), _c.c_longlong(T), H, K, int(ctx.safe), _c.c_float(ctx.lower),
                                       stream_ptr()), "kda_gate_bwd")
        return dx.to(ctx.dts[0]), dA.to(ctx.dts[1]), (db.to(ctx.dts[2]) if ctx.has_b else None), None, None


def kda_gate(x_g, A_log, dt_bias, safe_gate, lower_bound):
    return _KDAGate.apply(x_g, A_log, dt_bias, bool(safe_gate), float(lower_bound))


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, theta):
        T, H, dh = x.shape
        x2 = _bf(x).contiguous()
        out = torch.empty_like(x2)
        check(lib().hippo_rope(ptr(x2), ptr(out), ptr(pos), _c.c_longlong(T), H, dh, _c.c_float(theta),
                               _c.c_float(1.0), stream_ptr()), "rope")
        ctx.save_for_backward(pos)
        ctx.theta = theta
        return out

    @staticmethod
    def backward(ctx, dy):
        (pos,) = ctx.saved_tensors
        T, H, dh = dy.shape
        d2 = _bf(dy).contiguous()
        out = torch.empty_like(d2)
        check(lib().hippo_rope(ptr(d2), ptr(out), ptr(pos), _c.c_longlong(T), H, dh, _c.c_float(ctx.theta),
                               _c.c_float(-1.0), stream_ptr()), "rope_bwd")
        return out, None, None


def rope(q, k, positions, theta):
    pos = positions.to(torch.int32).contiguous()
    return _Rope.apply(q, pos, theta), _Rope.apply(k, pos, theta)


class _ShortConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, pos):
        T, D = x.shape
        W = weight.shape[1]
        xb = _bf(x)
        if xb.stride(1) != 1:
            xb = xb.contiguous()
        wb = _bf(weight).contiguous()
        y = torch.empty((T, D), dtype=torch.bfloat16, device=x.device)
        check(lib().hippo_short_conv_fwd(ptr(xb), _c.c_longlong(xb.stride(0)), ptr(wb), ptr(pos), ptr(y), _c.c_longlong(T),
                                         D, W, stream_ptr()), "short_conv_fwd")
        ctx.save_for_backward(xb, wb, pos)
        ctx.wdtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xb, wb, pos = ctx.saved_tensors
        T, D = dy.shape
        W = wb.shape[1]
        dy = _bf(dy).contiguous()
        dx = torch.empty((T, D), dtype=torch.bfloat16, device=dy.device)
        dw = torch.zeros((D, W), dtype=torch.float32, device=dy.device)
        check(lib().hippo_short_conv_bwd(ptr(xb), _c.c_longlong(xb.stride(0)), ptr(wb), ptr(pos), ptr(dy), ptr(dx),
                                         _c.c_longlong(D), ptr(dw), _c.c_longlong(T), D, W, stream_ptr()), "short_conv_bwd")
        return dx, dw.to(ctx.wdtype), None


def short_conv_silu(x, weight, bias, cu_seqlens):
    assert bias is None, "conv_bias is not supported on the CUDA path"
    from ..ref.ops import positions_from_cu
    pos = positions_from_cu(cu_seqlens, x.shape[0], x.device).to(torch.int32).contiguous()
    return _ShortConv.apply(x, weight, pos)


# ----------------------------------------------------------------------------- attention / KDA / AttnRes
class _KDAPrologue(torch.autograd.Function):
    """q / k / v / beta from the fused projection, plus (``fg_w`` > 0) a contiguous copy of the ``fg_w`` columns at
    ``off_fg`` (the inputs of the low-rank gate projections): their gradient comes back here and is written into the
    one projection gradient, instead of a zero-filled full-width tensor per slice plus an add."""

    @staticmethod
    def forward(ctx, proj, H, K, off_q, off_k, off_v, off_b, scale, beta_mul, apply_silu, off_fg, fg_w):
        proj = _bf(proj).contiguous()
        T, ld = proj.shape
        dev = proj.device
        q, k, v = (torch.empty((T, H, K), dtype=torch.bfloat16, device=dev) for _ in range(3))
        beta, qr, kr = (torch.empty((T, H), dtype=torch.float32, device=dev) for _ in range(3))
        check(lib().hippo_kda_prologue_fwd(ptr(proj), _c.c_longlong(ld), H, K, off_q, off_k, off_v, off_b, ptr(q),
                                           ptr(k), ptr(v), ptr(beta), ptr(qr), ptr(kr), _c.c_longlong(T),
                                           _c.c_float(scale), _c.c_float(beta_mul), int(apply_silu), stream_ptr()),
              "kda_prologue_fwd")
        ctx.save_for_backward(proj, qr, kr)
        ctx.meta = (H, K, off_q, off_k, off_v, off_b, scale, beta_mul, apply_silu, off_fg, fg_w)
        fg = proj[:, off_fg:off_fg + fg_w].contiguous() if fg_w > 0 else proj.new_empty((T, 0))
        return q, k, v, beta, fg

    @staticmethod
    def backward(ctx, dq, dk, dv, dbeta, dfg):
        proj, qr, kr = ctx.saved_tensors
        H, K, off_q, off_k, off_v, off_b, scale, beta_mul, apply_silu, off_fg, fg_w = ctx.meta
        T, ld = proj.shape
        dev = proj.device
        # the kernel writes the q, k, v and beta columns; the gate columns and whatever else the projection carries
        # (padding) are filled here
        covered = sorted([(off_q, H * K), (off_k, H * K), (off_v, H * K), (off_b, H)] + ([(off_fg, fg_w)] if fg_w > 0 else []))
        dproj = torch.empty_like(proj)
        pos = 0
        for o, n in covered:
            if o > pos:
                dproj[:, pos:o].zero_()
            pos = max(pos, o + n)
        if pos < ld:
            dproj[:, pos:].zero_()
        if fg_w > 0:
            if dfg is not None:
                dproj[:, off_fg:off_fg + fg_w].copy_(dfg)
            else:
                dproj[:, off_fg:off_fg + fg_w].zero_()
        bf = dict(dtype=torch.bfloat16, device=dev)
        dq = _bf(dq).contiguous() if dq is not None else torch.zeros((T, H, K), **bf)
        dk = _bf(dk).contiguous() if dk is not None else torch.zeros((T, H, K), **bf)
        dv = _bf(dv).contiguous() if dv is not None else torch.zeros((T, H, K), **bf)
        dbeta = dbeta.float().contiguous() if dbeta is not None else torch.zeros((T, H), device=dev)
        check(lib().hippo_kda_prologue_bwd(ptr(proj), _c.c_longlong(ld), H, K, off_q, off_k, off_v, off_b, ptr(dq),
                                           ptr(dk), ptr(dv), ptr(dbeta), ptr(qr), ptr(kr), ptr(dproj),
                                           _c.c_longlong(T), _c.c_float(scale), _c.c_float(beta_mul),
                                           int(apply_silu), stream_ptr()), "kda_prologue_bwd")
        return (dproj,) + (None,) * 11


def kda_prologue(proj, H, K, off_q, off_k, off_v, off_b, scale, beta_mul, apply_silu, off_fg=0, fg_w=0):
    out = _KDAPrologue.apply(proj, H, K, off_q, off_k, off_v, off_b, float(scale), float(beta_mul), bool(apply_silu),
                             int(off_fg), int(fg_w))
    return out if fg_w > 0 else out[:4]


def kda(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_qk_l2norm, skip_saved=False, mode="chunk"):
    from . import kda_cuda
    return kda_cuda.kda(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_qk_l2norm, skip_saved, mode)


def causal_attention(q, k, v, cu_seqlens, scale):
    from . import attn_cuda
    return attn_cuda.causal_attention(q, k, v, cu_seqlens, scale)


def attn_res(sources, query, norm_weight, eps):
    from . import attnres_cuda
    return attnres_cuda.attn_res(sources, query, norm_weight, eps)


# ----------------------------------------------------------------------------- NVFP4
def nvfp4_quantize(w, global_scale=None):
    from . import nvfp4_cuda
    return nvfp4_cuda.quantize(w, global_scale)


def nvfp4_dequantize(packed, scales, global_scale, dtype=torch.float32):
    from . import nvfp4_cuda
    return nvfp4_cuda.dequantize(packed, scales, global_scale, dtype)


def nvfp4_gemm_nt(x, packed, scales, global_scale, act_quant=True, act_gs=None):
    from . import nvfp4_cuda
    return nvfp4_cuda.gemm_nt(x, packed, scales, global_scale, act_quant, act_gs)


# ----------------------------------------------------------------------------- optimizer math
def newton_schulz5(G, steps=5, eps=1e-7):
    """Quintic Newton-Schulz on the tcgen05 GEMM: S = X X^T (NT), S2 = S S, X <- a X + (b S + c S2) X."""
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.float()
    X = (X / (X.norm() + eps)).to(torch.bfloat16)
    tall = X.shape[0] > X.shape[1]
    if tall:
        X = X.t().contiguous()
    n = X.shape[0]
    if n % 8 or X.shape[1] % 8:
        from ..ref.ops import newton_schulz5 as ref_ns
        return ref_ns(G, steps, eps)
    for _ in range(steps):
        S = gemm_nt(X, X)                                # [n, n]
        S2 = gemm_nn(S, S)
        M = (b * S.float() + c * S2.float()).to(torch.bfloat16)
        X = (a * X.float() + gemm_nn(M, X).float()).to(torch.bfloat16)
    if tall:
        X = X.t()
    return X.float()


def adamw_update(p, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    from . import optim_cuda
    return optim_cuda.adamw_update(p, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale)


def lce_chunk_stats(x, w, targets_local):
    z = gemm_nt(x, w, out_dtype=torch.float32)
    C, V = z.shape
    mx, se, tz = (torch.empty(C, dtype=torch.float32, device=z.device) for _ in range(3))
    tg = targets_local.to(torch.int64).contiguous()
    check(lib().hippo_ce_stats(ptr(z), ptr(tg), ptr(mx), ptr(se), ptr(tz), _c.c_longlong(C), V, stream_ptr()), "ce_stats")
    return z, mx, se, tz


def lce_chunk_grad(z, lse, targets_local, row_weight):
    """dz = (softmax(z) - onehot) * row_weight as bf16 (z: fp32 logits of this vocab shard)."""
    C, V = z.shape
    dz = torch.empty((C, V), dtype=torch.bfloat16, device=z.device)
    tg = targets_local.to(torch.int64).contiguous()
    check(lib().hippo_ce_grad(ptr(z), ptr(lse.float().contiguous()), ptr(tg), ptr(row_weight.float().contiguous()),
                              ptr(dz), _c.c_longlong(C), V, stream_ptr()), "ce_grad")
    return dz


def lce_epilogue_supported(x, w) -> bool:
    """The logits GEMM with statistics in its epilogue stores bf16 logits: bf16 activations only (an fp32 run keeps fp32
    logits), 16-byte aligned rows on both operands and the output."""
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0


def lce_logits_stats(x, w, targets_local):
    """z = x @ w^T stored as bf16, with the softmax statistics taken from the accumulator in the GEMM epilogue
    (``hippo_gemm_bf16_lce``): returns (z [C, V] bf16, part [ceil(V/256), C, 2] fp32 = per 256-column tile (max, sum exp)
    of the stored logits, tz [C] fp32 = logit at the target column (undefined where the target is -1), targets as int64)."""
    C, K = x.shape
    V = w.shape[0]
    x = x.to(torch.bfloat16)
    w = w.to(torch.bfloat16)
    if x.stride(-1) != 1 or (x.stride(0) % 8) or (x.data_ptr() % 16):
        x = x.contiguous()
    if w.stride(-1) != 1 or (w.stride(0) % 8) or (w.data_ptr() % 16):
        w = w.contiguous()
    z = torch.empty((C, V), dtype=torch.bfloat16, device=x.device)
    part = torch.empty(((V + 255) // 256, C, 2), dtype=torch.float32, device=x.device)
    tz = torch.empty(C, dtype=torch.float32, device=x.device)
    tg = targets_local.to(torch.int64).contiguous()
    check(lib().hippo_gemm_bf16_lce(ptr(x), ptr(w), ptr(z), ptr(part), ptr(tg), ptr(tz), C, V, K,
                                    _c.c_longlong(x.stride(0)), _c.c_longlong(w.stride(0)), _c.c_longlong(V),
                                    stream_ptr()), "gemm_bf16_lce")
    return z, part, tz, tg


def lce_grad_inplace_local(z, part, tz, tg, row_weight, loss_sum):
    """Single-rank tail of ``lce_logits_stats``: merges the per-tile statistics of every row, overwrites the bf16 logits
    ``z`` with dz = (softmax - onehot) * row_weight and adds sum(lse - z_target) of weighted rows to ``loss_sum`` (fp32[1])."""
    C, V = z.shape
    stats = torch.empty((C, 4), dtype=torch.float32, device=z.device)
    sp = (_c.c_void_p * 1)(stats.data_ptr())
    check(lib().hippo_ce_part_merge(ptr(part), ptr(tz), ptr(tg), _c.c_longlong(C), part.shape[0], sp, None, 1, 0, C,
                                    stream_ptr()), "ce_part_merge")
    rw = row_weight.float().contiguous()
    check(lib().hippo_ce_grad_inplace(ptr(z), ptr(tg), ptr(rw), _c.c_longlong(C), V, ptr(loss_sum), sp, None, 1, 0, C,
                                      _c.c_uint(0), _c.c_longlong(0), stream_ptr()), "ce_grad_inplace")
    return z


def gemm_tn_accumulate(a, b, out_fp32):
    """out_fp32[N,K] += a[M,N]^T @ b[M,K] (fp32 accumulator tensor updated by the GEMM epilogue)."""
    Mc, N = a.shape
    K = b.shape[1]
    if N % 8 or K % 8:
        out_fp32 += (a.float().t() @ b.float())
        return out_fp32
    return _gemm(a.to(torch.bfloat16), b.to(torch.bfloat16), 2, N, K, Mc, out=out_fp32, accumulate=True)
