"""Data-parallel gradient reduction, overlapped with backward.

Each parameter gets a post-accumulate-grad hook; on the last micro-batch of a step the hook copies
the finished gradient into a flat bucket and, when the bucket is full, launches an asynchronous
all-reduce on the DP group (NCCL runs it on its own stream while backward continues).
``finish()`` waits for the outstanding buckets and scatters the sums back into ``p.grad``.
The loss is already normalised by the global valid-token count, so the reduction is a SUM.
With ``owners`` (gradient holder -> owning DP rank, from ``Muon.dp_owner_map``) the gradients of the
Muon matrices are REDUCED to their owner only (half the traffic of an all-reduce): the owner is the
only replica that uses them. Everything else is all-reduced.
The reference has no data parallelism (``scripts/train.py:216-237``: world == TP group).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.nvfp4_linear import NVFP4Linear


class DPGradReducer:
    def __init__(self, model: nn.Module, mesh, overlap: bool = True, bucket_mb: float = 256.0, owners=None):
        self.model, self.mesh, self.overlap = model, mesh, overlap
        self.bucket_elems = int(bucket_mb * 2 ** 20 / 2)
        self._last = True
        self._pending: List = []          # (work, flat, [tensors], owner)
        self.owners = owners or {}        # id(parameter | NVFP4 module) -> owning DP rank
        self._buckets = {}                # owner (None = all-reduce) -> [tensors]
        self._elems = {}
        self._hooked = False
        self._seen = set()                # ids of the gradients a hook has bucketed in this step
        if overlap and mesh.dp > 1:
            for p in model.parameters():
                if p.requires_grad:
                    p.register_post_accumulate_grad_hook(self._hook)
            self._hooked = True

    def set_last_microbatch(self, last: bool):
        self._last = last

    def _hook(self, p):
        if not self._last or p.grad is None:
            return
        self._seen.add(id(p))
        self._add(p.grad, self.owners.get(id(p)))

    def _add(self, g: torch.Tensor, owner=None):
        self._buckets.setdefault(owner, []).append(g)
        self._elems[owner] = self._elems.get(owner, 0) + g.numel()
        if self._elems[owner] >= self.bucket_elems:
            self._launch(owner)

    def _launch(self, owner=None):
        gs = self._buckets.get(owner)
        if not gs:
            return
        self._buckets[owner], self._elems[owner] = [], 0
        dt = torch.float32 if any(g.dtype == torch.float32 for g in gs) else gs[0].dtype
        if dist.get_backend(self.mesh.dp_group) == "gloo":
            dt = torch.float32
        flat = torch.cat([g.reshape(-1).to(dt) for g in gs])
        if owner is None:
            work = dist.all_reduce(flat, group=self.mesh.dp_group, async_op=True)
        else:
            work = dist.reduce(flat, dst=self.mesh.dp_ranks()[owner], group=self.mesh.dp_group, async_op=True)
        self._pending.append((work, flat, gs, owner))

    def finish(self):
        if self.mesh.dp == 1:
            return
        # everything a hook has not bucketed in this step (no hooks at all, or a gradient that was installed after
        # backward, e.g. uploaded from the host accumulators); every replica walks the parameters in the same order
        for p in self.model.parameters():
            if p.grad is not None and id(p) not in self._seen:
                self._add(p.grad, self.owners.get(id(p)))
        self._seen = set()
        for mod in self.model.modules():
            if isinstance(mod, NVFP4Linear) and mod.no_master and mod.grad_w is not None:
                self._add(mod.grad_w, self.owners.get(id(mod)))
        for owner in list(self._buckets):
            self._launch(owner)
        for work, flat, gs, owner in self._pending:
            work.wait()
            if owner is not None and owner != self.mesh.dp_rank:
                continue                      # only the owner holds (and uses) the reduced gradient
            off = 0
            for g in gs:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g)); off += n
        self._pending = []
