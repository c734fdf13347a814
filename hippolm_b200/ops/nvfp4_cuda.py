"""CUDA path of NVFP4 quantise / dequantise / block-scaled GEMM."""
from __future__ import annotations

import torch

from ..ref import ops as _ro


def quantize(w, global_scale=None):
    return _ro.nvfp4_quantize(w, global_scale)


def dequantize(packed, scales, global_scale, dtype=torch.float32):
    return _ro.nvfp4_dequantize(packed, scales, global_scale, dtype)


def gemm_nt(x, packed, scales, global_scale, act_quant=True):
    from . import cuda_ops
    w = dequantize(packed, scales, global_scale, torch.bfloat16)
    xq = x
    if act_quant:
        xq = dequantize(*quantize(x), dtype=torch.bfloat16)
    return cuda_ops.gemm_nt(xq, w)
