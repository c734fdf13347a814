"""CUDA path of NVFP4 quantise / dequantise (``csrc/misc_ops.cu``) and the block-scaled GEMM."""
from __future__ import annotations

import ctypes as _c

import torch

from ._ext import lib, ptr, stream_ptr, check


def quantize(w: torch.Tensor, global_scale=None):
    """[N, K] -> (packed u8 [N, K/2], e4m3 scales [N, K/16], fp32 global scale [1])."""
    N, K = w.shape
    assert K % 16 == 0
    x = w if w.dtype in (torch.bfloat16, torch.float32) else w.float()
    x = x.contiguous()
    packed = torch.empty((N, K // 2), dtype=torch.uint8, device=w.device)
    scales = torch.empty((N, K // 16), dtype=torch.uint8, device=w.device)
    compute = global_scale is None
    gs = torch.empty(1, dtype=torch.float32, device=w.device) if compute else global_scale.float().reshape(1).contiguous()
    scratch = torch.empty(1, dtype=torch.float32, device=w.device)
    check(lib().hippo_nvfp4_quantize(ptr(x), int(x.dtype == torch.bfloat16), _c.c_longlong(N), _c.c_longlong(K), ptr(gs),
                                     int(compute), ptr(scratch), ptr(packed), ptr(scales), stream_ptr()), "nvfp4_quantize")
    return packed, scales.view(torch.float8_e4m3fn), gs


def tensor_scale(x: torch.Tensor) -> torch.Tensor:
    """fp32 [1] tensor scale absmax(x) / (6 * 448) (1 for an all-zero tensor), computed on the device."""
    x = x if x.dtype in (torch.bfloat16, torch.float32) else x.float()
    x = x.contiguous()
    gs = torch.empty(1, dtype=torch.float32, device=x.device)
    scratch = torch.empty(1, dtype=torch.float32, device=x.device)
    check(lib().hippo_nvfp4_tensor_scale(ptr(x), _c.c_longlong(x.numel()), int(x.dtype == torch.bfloat16), ptr(scratch),
                                         ptr(gs), stream_ptr()), "nvfp4_tensor_scale")
    return gs


def quantize_transposed(x: torch.Tensor, global_scale=None):
    """x [T, C] bf16 -> NVFP4 of x^T with the 16-element blocks along T: (packed u8 [C, T/2], block scales already in the
    MMA tile layout (uint8, [ceil(C/128) * T/64 * 512]), fp32 tensor scale [1]). Operand of the weight-gradient product,
    whose contraction runs over the tokens."""
    T, C = x.shape
    assert T % 64 == 0 and C % 8 == 0 and x.dtype == torch.bfloat16 and x.stride(1) == 1
    gs = tensor_scale(x) if global_scale is None else global_scale.float().reshape(1).contiguous()
    packed = torch.empty((C, T // 2), dtype=torch.uint8, device=x.device)
    cp = (C + 127) // 128 * 128
    alloc = torch.zeros if cp != C else torch.empty
    sf = alloc(cp * (T // 16), dtype=torch.uint8, device=x.device)
    check(lib().hippo_nvfp4_quantize_transposed(ptr(x), _c.c_longlong(x.stride(0)), _c.c_longlong(T), C, ptr(gs),
                                                ptr(packed), ptr(sf), stream_ptr()), "nvfp4_quantize_transposed")
    return packed, sf, gs


def dequantize(packed, scales, global_scale, dtype=torch.float32):
    N, K2 = packed.shape
    K = K2 * 2
    od = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    out = torch.empty((N, K), dtype=od, device=packed.device)
    sc = scales.view(torch.uint8).contiguous()
    check(lib().hippo_nvfp4_dequantize(ptr(packed.contiguous()), ptr(sc), ptr(global_scale.float().contiguous()), ptr(out),
                                       int(od == torch.bfloat16), _c.c_longlong(N), _c.c_longlong(K), stream_ptr()),
          "nvfp4_dequantize")
    return out if od == dtype else out.to(dtype)


def gemm_nt(x, packed, scales, global_scale, act_quant=True, act_gs=None):
    """y = Q(x) dq(W)^T."""
    from . import fp4_gemm
    return fp4_gemm.gemm_nt(x, packed, scales, global_scale, act_quant, act_gs)
