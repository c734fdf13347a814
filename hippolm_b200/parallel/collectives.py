"""Collectives with correct conjugate backward rules.

The reference's wrappers (``src/models/tp_model/_primitives.py:148-247``) have identity
backward for all-reduce and no backward collective for column-parallel inputs; here each
forward collective carries its true adjoint:

  gather_seq          all-gather(dim 0)      <->  reduce-scatter(dim 0)
  reduce_scatter_seq  reduce-scatter(dim 0)  <->  all-gather(dim 0)
  copy_to_tp          identity               <->  all-reduce
  reduce_from_tp      all-reduce             <->  identity
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .mesh import get_mesh


def _backend_of(group) -> str:
    try:
        return dist.get_backend(group)
    except Exception:
        return "gloo"


def all_gather_dim0(x: torch.Tensor, group, world: int) -> torch.Tensor:
    if world == 1:
        return x
    x = x.contiguous()
    out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def reduce_scatter_dim0(x: torch.Tensor, group, world: int) -> torch.Tensor:
    if world == 1:
        return x
    x = x.contiguous()
    assert x.shape[0] % world == 0, f"dim0 {x.shape[0]} not divisible by {world}"
    n = x.shape[0] // world
    if _backend_of(group) == "gloo":
        # gloo has no reduce_scatter: all-reduce then slice (CPU test path only)
        y = x.clone()
        if y.dtype == torch.bfloat16:
            yf = y.float(); dist.all_reduce(yf, group=group); y = yf.to(torch.bfloat16)
        else:
            dist.all_reduce(y, group=group)
        r = dist.get_rank(group)
        return y[r * n:(r + 1) * n].contiguous()
    out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


def all_reduce_sum(x: torch.Tensor, group, world: int) -> torch.Tensor:
    if world == 1:
        return x
    x = x.contiguous()
    if _backend_of(group) == "gloo" and x.dtype == torch.bfloat16:
        xf = x.float(); dist.all_reduce(xf, group=group); x.copy_(xf)
        return x
    dist.all_reduce(x, group=group)
    return x


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        m = get_mesh()
        return all_gather_dim0(x, m.tp_group, m.tp)

    @staticmethod
    def backward(ctx, g):
        m = get_mesh()
        return reduce_scatter_dim0(g, m.tp_group, m.tp)


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        m = get_mesh()
        return reduce_scatter_dim0(x, m.tp_group, m.tp)

    @staticmethod
    def backward(ctx, g):
        m = get_mesh()
        return all_gather_dim0(g, m.tp_group, m.tp)


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        m = get_mesh()
        return all_reduce_sum(g.clone(), m.tp_group, m.tp)


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        m = get_mesh()
        return all_reduce_sum(x.clone(), m.tp_group, m.tp)

    @staticmethod
    def backward(ctx, g):
        return g


def gather_seq(x):
    return x if get_mesh().tp == 1 else _GatherSeq.apply(x)


def reduce_scatter_seq(x):
    return x if get_mesh().tp == 1 else _ReduceScatterSeq.apply(x)


def copy_to_tp(x):
    return x if get_mesh().tp == 1 else _CopyToTP.apply(x)


def reduce_from_tp(x):
    return x if get_mesh().tp == 1 else _ReduceFromTP.apply(x)


def sync_replicated_grads(params, mesh=None) -> None:
    """All-reduce (SUM) the gradients of TP-replicated parameters.

    Under sequence parallelism every rank sees T/tp tokens (norm weights, AttnRes query)
    or a column-parallel partial (``fg_first``), so the replicas' gradients are partial
    sums. The reference never syncs them and its replicas drift at world>1.
    """
    m = mesh or get_mesh()
    if m.tp == 1:
        return
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=m.tp_group)
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off:off + n].view_as(g))
        off += n


def broadcast_replicated_params(params, mesh=None) -> None:
    """Make TP-replicated parameters bit-identical (source = tp_rank 0 of each group)."""
    m = mesh or get_mesh()
    if m.tp == 1:
        return
    src = m.tp_ranks()[0]
    for p in params:
        dist.broadcast(p.data, src=src, group=m.tp_group)
