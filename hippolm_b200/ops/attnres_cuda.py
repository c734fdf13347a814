"""CUDA path of the block attention residual mix."""
from __future__ import annotations

import torch

from ..ref.ops import attn_res as _ref


def attn_res(sources, query, norm_weight, eps):
    return _ref(torch.stack(sources, 0), query, norm_weight, eps)
