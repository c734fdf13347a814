"""Block-scaled NVFP4 GEMM entry point (``csrc/gemm_fp4.cu``): y = Q(x) dq(W)^T on the FP4 tensor cores."""
from __future__ import annotations

import ctypes as C
import os

import torch

from ._ext import lib, ptr, stream_ptr, check


def tile_scales(scales: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """logical e4m3 scales [rows, K/16] -> the 512-byte (128 rows x 4 k-groups) tiles the MMA reads."""
    rp = (rows + 127) // 128 * 128
    out = torch.empty(rp * (K // 16), dtype=torch.uint8, device=scales.device)
    check(lib().hippo_nvfp4_tile_scales(ptr(scales.view(torch.uint8).contiguous()), ptr(out), C.c_longlong(rows),
                                        C.c_longlong(K), stream_ptr()), "nvfp4_tile_scales")
    return out


_EPOCH = [0]            # bumped whenever a stored NVFP4 weight is rewritten (NVFP4Linear.weight_changed)
_TILED = {}             # id(scales tensor) -> (weakref to it, epoch, tiled scales)


def weights_changed() -> None:
    """Called by every writer of a stored NVFP4 weight: tiled copies of weight scales are rebuilt at their next use."""
    _EPOCH[0] += 1


def tile_weight_scales(scales: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """``tile_scales`` for the scales of a WEIGHT, cached while the very same tensor object is alive and no stored weight
    has been rewritten: the re-tiling then runs once per optimizer step instead of once per GEMM call. Temporaries
    (freshly quantised master weights) never hit: their tensor objects die with the call."""
    import weakref
    hit = _TILED.get(id(scales))
    if hit is not None and hit[0]() is scales and hit[1] == _EPOCH[0]:
        return hit[2]
    tiled = tile_scales(scales, rows, K)
    if len(_TILED) > 4096:
        _TILED.clear()
    _TILED[id(scales)] = (weakref.ref(scales), _EPOCH[0], tiled)
    return tiled


def fp4_matmul(a_packed, a_scales, a_gs, b_packed, b_scales, b_gs) -> torch.Tensor:
    """[M, K/2] x [N, K/2]^T with logical scales [*, K/16] and fp32 tensor scales -> bf16 [M, N]. ``b`` is the weight."""
    M, K2 = a_packed.shape
    N = b_packed.shape[0]
    K = K2 * 2
    sfa, sfb = tile_scales(a_scales, M, K), tile_weight_scales(b_scales, N, K)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=a_packed.device)
    check(lib().hippo_gemm_nvfp4(ptr(a_packed), ptr(b_packed), ptr(sfa), ptr(sfb), ptr(a_gs), ptr(b_gs), ptr(out),
                                 M, N, K, C.c_longlong(N), stream_ptr()), "gemm_nvfp4")
    return out


def fp4_matmul_tiled(a_packed, sfa_tiled, a_gs, b_packed, sfb_tiled, b_gs, out=None, accumulate: bool = False) -> torch.Tensor:
    """Same product with block scales that are already in the MMA tile layout; ``accumulate`` adds into ``out`` (bf16)."""
    M, K2 = a_packed.shape
    N = b_packed.shape[0]
    K = K2 * 2
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a_packed.device)
    assert out.dtype == torch.bfloat16 and out.shape == (M, N) and out.stride(1) == 1
    fn = lib().hippo_gemm_nvfp4_accumulate if accumulate else lib().hippo_gemm_nvfp4
    check(fn(ptr(a_packed), ptr(b_packed), ptr(sfa_tiled), ptr(sfb_tiled), ptr(a_gs), ptr(b_gs), ptr(out), M, N, K,
             C.c_longlong(out.stride(0)), stream_ptr()), "gemm_nvfp4")
    return out


def fp4_matmul_pair(a_packed, sfa_tiled, a_gs, b_packed, sfb_tiled, b_gs, out=None, accumulate: bool = False) -> torch.Tensor:
    """The same product on the CTA-pair kernel (``csrc/gemm_fp4_2sm.cu``: 256 x 256 tiles, ``cta_group::2``), called
    explicitly; ``fp4_matmul`` / ``fp4_matmul_tiled`` reach it through the library unless ``HIPPO_FP4_PAIR=0``.
    Needs at least 256 rows and 256 columns."""
    M, K2 = a_packed.shape
    N = b_packed.shape[0]
    K = K2 * 2
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a_packed.device)
    assert out.dtype == torch.bfloat16 and out.shape == (M, N) and out.stride(1) == 1
    check(lib().hippo_gemm_nvfp4_pair(ptr(a_packed), ptr(b_packed), ptr(sfa_tiled), ptr(sfb_tiled), ptr(a_gs), ptr(b_gs),
                                      ptr(out), M, N, K, C.c_longlong(out.stride(0)), int(bool(accumulate)), stream_ptr()),
          "gemm_nvfp4_pair")
    return out


def supported(M: int, N: int, K: int) -> bool:
    return K % 256 == 0 and N % 8 == 0 and os.environ.get("HIPPO_FP4_GEMM", "1") != "0"


def gemm_nt(x, packed, scales, global_scale, act_quant=True, act_gs=None):
    """``act_gs``: tensor scale of ``x`` when the caller already knows it (saves the absmax pass over ``x``)."""
    from . import cuda_ops, nvfp4_cuda
    M, K = x.shape
    N = packed.shape[0]
    if act_quant and supported(M, N, K):
        xp, xs, xg = nvfp4_cuda.quantize(x.contiguous(), act_gs)
        return fp4_matmul(xp, xs, xg, packed, scales, global_scale.float().contiguous())
    w = nvfp4_cuda.dequantize(packed, scales, global_scale, torch.bfloat16)
    xq = nvfp4_cuda.dequantize(*nvfp4_cuda.quantize(x), dtype=torch.bfloat16) if act_quant else x
    return cuda_ops.gemm_nt(xq, w)
