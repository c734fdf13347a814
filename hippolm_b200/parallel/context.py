"""Context parallelism for the KDA recurrence: one long sequence split into contiguous token segments across the
ranks of a process group.

The delta-rule state update is linear in the state, so a segment acts on its incoming state as
``S_end = M S_start + U`` with a transition ``M`` [H, K, K] that depends only on (k, g, beta) and an offset
``U`` [H, K, V]. Every rank computes (M, U) of its own segment (two local passes: the recurrence on the K unit
vectors with v = 0 gives M, the recurrence from a zero state gives U), the pairs are all-gathered, each rank folds
the pairs of the ranks before it into its incoming state, and a third local pass produces the outputs. Gradients flow
through the gathered pairs (the backward of the gather is a sum over ranks), so the result matches the single-device
recurrence for q, k, v, g and beta alike.

This is the scheme the reference carries as dormant vendored code (``fla/ops/cp/chunk_delta_h.py:797-880``: per-rank
end state + transition, all-gather, prefix merge; ``fla/ops/cp/context.py:22-172``) and never enables. Here it is an
option for sequences longer than one rank wants to hold; the training loop's default for long sequences stays
micro-batching with carried state.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops


class _AllGatherStack(torch.autograd.Function):
    """x -> stack of every rank's x along a new leading axis; backward: sum over ranks of the slot this rank filled."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        outs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(outs, x.contiguous(), group=group)
        return torch.stack(outs, 0)

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        dist.all_reduce(grad, group=ctx.group)
        return grad[dist.get_rank(ctx.group)], None


def kda_context_parallel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                         group, scale: Optional[float] = None, initial_state: Optional[torch.Tensor] = None,
                         use_qk_l2norm: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """q, k, g: [T_local, H, K]; v: [T_local, H, V]; beta: [T_local, H]: this rank's segment of ONE sequence
    (rank r of ``group`` holds the r-th segment). ``initial_state`` [1, H, K, V] is the state before the first
    segment (same on every rank). Returns (o [T_local, H, V], final state of the whole sequence [1, H, K, V])."""
    cp, r = dist.get_world_size(group), dist.get_rank(group)
    T, H, K = q.shape
    V = v.shape[-1]
    # offset: end state of the local segment from a zero start
    _, U = ops.kda(q, k, v, g, beta, scale, None, None, use_qk_l2norm)
    # transition: the same recurrence applied to the K unit vectors (v = 0 leaves only the decay / erase terms)
    eye = torch.eye(K, dtype=torch.float32, device=q.device).expand(1, H, K, K).contiguous()
    _, M = ops.kda(q, k, torch.zeros(T, H, K, dtype=v.dtype, device=v.device), g, beta, scale, eye, None, use_qk_l2norm)
    Us = _AllGatherStack.apply(U.float(), group)              # [cp, 1, H, K, V]
    Ms = _AllGatherStack.apply(M.float(), group)              # [cp, 1, H, K, K]
    S = initial_state.float() if initial_state is not None else torch.zeros(1, H, K, V, dtype=torch.float32, device=q.device)
    S_in = S
    for j in range(cp):
        if j == r:
            S_in = S
        S = Ms[j] @ S + Us[j]
    o, _ = ops.kda(q, k, v, g, beta, scale, S_in, None, use_qk_l2norm)
    return o, S
