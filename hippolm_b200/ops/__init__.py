"""Op surface used by the model code.

Every op has exactly two implementations: the sm_100a kernels in ``hippolm_b200/csrc``
(taken whenever the tensors live on a CUDA device; a missing extension raises) and the
pure-torch oracle in ``hippolm_b200/ref`` (taken for CPU tensors). There is no backend
registry (the reference's ``fla/ops/backends/__init__.py:30-201`` dispatch has no counterpart).
"""
from .functional import (  # noqa: F401
    gemm_nt, gemm_nn, gemm_tn, linear, rmsnorm, add_rmsnorm, swiglu, gated_rmsnorm, kda, kda_gate, kda_prologue,
    short_conv_silu, rope, causal_attention, attention_decode, attn_res, l2norm, silu,
    nvfp4_quantize, nvfp4_dequantize, nvfp4_linear, newton_schulz5, adamw_update,
    lce_chunk_stats, lce_chunk_grad, gemm_tn_accumulate, cuda_ext_loaded,
)
