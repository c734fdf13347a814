"""Block-scaled NVFP4 GEMM entry point."""
from __future__ import annotations

import torch


def gemm_nt(x, packed, scales, global_scale, act_quant=True):
    from . import cuda_ops, nvfp4_cuda
    w = nvfp4_cuda.dequantize(packed, scales, global_scale, torch.bfloat16)
    xq = x
    if act_quant:
        xq = nvfp4_cuda.dequantize(*nvfp4_cuda.quantize(x), dtype=torch.bfloat16)
    return cuda_ops.gemm_nt(xq, w)
