"""CUDA path of causal varlen attention."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def causal_attention(q, k, v, cu_seqlens, scale):
    T, H, dh = q.shape
    cu = [0, T] if cu_seqlens is None else [int(x) for x in cu_seqlens.tolist()]
    outs = []
    for s, e in zip(cu[:-1], cu[1:]):
        if e <= s:
            continue
        o = F.scaled_dot_product_attention(q[s:e].transpose(0, 1).unsqueeze(0), k[s:e].transpose(0, 1).unsqueeze(0),
                                           v[s:e].transpose(0, 1).unsqueeze(0), is_causal=True, scale=scale)
        outs.append(o.squeeze(0).transpose(0, 1))
    return torch.cat(outs, 0)
