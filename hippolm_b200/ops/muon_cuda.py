"""Device-side Muon: fused momentum/nesterov/norm kernel, Newton-Schulz on the tcgen05 GEMM with the
polynomial folded into the GEMM epilogues (``C = alpha*A*B + beta*Cin``), fused parameter update
(bf16 weights, or NVFP4 dequantise -> update -> re-quantise in one pass)."""
from __future__ import annotations

import ctypes as C

import torch

from ._ext import lib, ptr, stream_ptr, check

_A, _B, _C = 3.4445, -4.7750, 2.0315


def _gemm_ex(a, b, out, cin, M, N, K, layout, alpha, beta):
    check(lib().hippo_gemm_bf16_ex(ptr(a), ptr(b), ptr(out), ptr(cin), M, N, K, C.c_longlong(a.stride(0)),
                                   C.c_longlong(b.stride(0)), C.c_longlong(out.stride(0)),
                                   C.c_longlong(cin.stride(0) if cin is not None else 0), layout, C.c_float(alpha),
                                   C.c_float(beta), stream_ptr()), "gemm_bf16_ex")


def _gemm_sym(a, b, out, cin, n, K, layout, alpha, beta):
    """Square symmetric product (X X^T, X^T X, c S S + b S): only the tiles on or below the diagonal are computed by the
    CTA-pair kernel and then mirrored, which halves the cost of these steps."""
    check(lib().hippo_gemm_bf16_sym(ptr(a), ptr(b), ptr(out), ptr(cin), n, K, C.c_longlong(a.stride(0)),
                                    C.c_longlong(b.stride(0)), C.c_longlong(out.stride(0)),
                                    C.c_longlong(cin.stride(0) if cin is not None else 0), layout, C.c_float(alpha),
                                    C.c_float(beta), stream_ptr()), "gemm_bf16_sym")


_SYM_MIN = 512          # below this the mirror pass costs more than the skipped tiles


def supported(rows: int, cols: int) -> bool:
    return rows % 8 == 0 and cols % 8 == 0 and (rows * cols) % 8 == 0


def momentum_update(g: torch.Tensor, m: torch.Tensor, beta: float, gscale: float, nesterov: bool):
    """m <- beta m + g*gscale (in place); returns (u bf16, sum(u^2) device scalar)."""
    assert g.is_contiguous() and m.is_contiguous()
    u = torch.empty(g.shape, dtype=torch.bfloat16, device=g.device)
    ssq = torch.empty(1, dtype=torch.float32, device=g.device)
    check(lib().hippo_muon_momentum(ptr(g), int(g.dtype == torch.bfloat16), ptr(m), int(m.dtype == torch.bfloat16), ptr(u),
                                    C.c_longlong(g.numel()), C.c_float(beta), C.c_float(gscale), int(nesterov), ptr(ssq),
                                    stream_ptr()), "muon_momentum")
    return u, ssq


def newton_schulz_(u: torch.Tensor, ssq: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Orthogonalise u (bf16 [rows, cols], overwritten) given sum(u^2); returns the result (bf16)."""
    rows, cols = u.shape
    check(lib().hippo_scale_inv_norm(ptr(u), C.c_longlong(u.numel()), ptr(ssq), C.c_float(eps), stream_ptr()),
          "scale_inv_norm")
    n = min(rows, cols)
    S = torch.empty((n, n), dtype=torch.bfloat16, device=u.device)
    Mm = torch.empty((n, n), dtype=torch.bfloat16, device=u.device)
    X, Xn = u, torch.empty_like(u)
    for _ in range(steps):
        sym = n >= _SYM_MIN
        if rows <= cols:
            if sym:
                _gemm_sym(X, X, S, None, n, cols, 0, 1.0, 0.0)               # S = X X^T  (lower tiles + mirror)
                _gemm_sym(S, S, Mm, S, n, n, 1, _C, _B)                      # M = c S S + b S
            else:
                _gemm_ex(X, X, S, None, n, n, cols, 0, 1.0, 0.0)
                _gemm_ex(S, S, Mm, S, n, n, n, 1, _C, _B)
            _gemm_ex(Mm, X, Xn, X, rows, cols, n, 1, 1.0, _A)                # X' = M X + a X
        else:
            if sym:
                _gemm_sym(X, X, S, None, n, rows, 2, 1.0, 0.0)               # S = X^T X
                _gemm_sym(S, S, Mm, S, n, n, 1, _C, _B)
            else:
                _gemm_ex(X, X, S, None, n, n, rows, 2, 1.0, 0.0)
                _gemm_ex(S, S, Mm, S, n, n, n, 1, _C, _B)
            _gemm_ex(X, Mm, Xn, X, rows, cols, n, 1, 1.0, _A)                # X' = X M + a X
        X, Xn = Xn, X
    return X


def apply_update(w: torch.Tensor, o: torch.Tensor, wd_factor: float, lr: float) -> None:
    """w <- w*wd_factor - lr*o in place (w bf16/fp32 contiguous rows, o bf16)."""
    check(lib().hippo_axpby_update(ptr(w), int(w.dtype == torch.bfloat16), ptr(o), C.c_longlong(w.numel()),
                                   C.c_float(wd_factor), C.c_float(lr), stream_ptr()), "axpby_update")


def nvfp4_apply_update(mod, segments, wd_factor: float, lr: float, seed: int, stochastic: bool = True) -> None:
    """In-place update of a no-master NVFP4 weight: ``segments`` = [(row0, row1, o bf16 [row1-row0, K])] covering the
    rows that change. Three passes on the device and no host sync: absmax of the updated values over all segments,
    tensor scale from it, re-quantisation (block scales rounded up, stochastic E2M1 rounding) against the new scale."""
    packed, scales, gs = mod.packed_weight, mod.scales.view(torch.uint8), mod.global_scale
    K = packed.shape[1] * 2
    whole = sum(b - a for a, b, _ in segments) == packed.shape[0]
    tmp = torch.zeros(2, dtype=torch.float32, device=packed.device)          # [absmax, new tensor scale]
    amax, gs_new = tmp[0:1], tmp[1:2]
    if whole:
        for a, b, o in segments:
            check(lib().hippo_nvfp4_update_absmax(ptr(packed[a:b]), ptr(scales[a:b]), ptr(gs), ptr(o), C.c_longlong(b - a),
                                                  C.c_longlong(K), C.c_float(wd_factor), C.c_float(lr), ptr(amax),
                                                  stream_ptr()), "nvfp4_update_absmax")
        check(lib().hippo_nvfp4_scale_from_absmax(ptr(amax), ptr(gs_new), stream_ptr()), "nvfp4_scale_from_absmax")
    else:
        gs_new = gs                # a partial update cannot move the tensor scale of the rows it does not touch
    for a, b, o in segments:
        check(lib().hippo_nvfp4_apply_update(ptr(packed[a:b]), ptr(scales[a:b]), ptr(gs), ptr(gs_new), ptr(o),
                                             C.c_longlong(b - a), C.c_longlong(K), C.c_longlong(a * (K // 16)),
                                             C.c_float(wd_factor), C.c_float(lr), C.c_uint(seed & 0xFFFFFFFF),
                                             1 if stochastic else 0, stream_ptr()), "nvfp4_apply_update")
    if whole:
        gs.copy_(gs_new)
    mod.weight_changed()
