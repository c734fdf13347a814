"""Data-parallel gradient reduction, overlapped with backward.

Each parameter gets a post-accumulate-grad hook; on the last micro-batch of a step the hook copies
the finished gradient into a flat bucket and, when the bucket is full, launches an asynchronous
all-reduce on the DP group (NCCL runs it on its own stream while backward continues).
``finish()`` waits for the outstanding buckets and scatters the sums back into ``p.grad``.
The loss is already normalised by the global valid-token count, so the reduction is a SUM.
The reference has no data parallelism (``scripts/train.py:216-237``: world == TP group).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.nvfp4_linear import NVFP4Linear


class DPGradReducer:
    def __init__(self, model: nn.Module, mesh, overlap: bool = True, bucket_mb: float = 256.0):
        self.model, self.mesh, self.overlap = model, mesh, overlap
        self.bucket_elems = int(bucket_mb * 2 ** 20 / 2)
        self._last = True
        self._pending: List = []          # (work, flat, [(tensor, offset, numel)])
        self._cur: List = []
        self._cur_elems = 0
        self._hooked = False
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
        self._add(p.grad)

    def _add(self, g: torch.Tensor):
        self._cur.append(g)
        self._cur_elems += g.numel()
        if self._cur_elems >= self.bucket_elems:
            self._launch()

    def _launch(self):
        if not self._cur:
            return
        gs = self._cur
        self._cur, self._cur_elems = [], 0
        dt = torch.float32 if any(g.dtype == torch.float32 for g in gs) else gs[0].dtype
        if dist.get_backend(self.mesh.dp_group) == "gloo":
            dt = torch.float32
        flat = torch.cat([g.reshape(-1).to(dt) for g in gs])
        work = dist.all_reduce(flat, group=self.mesh.dp_group, async_op=True)
        self._pending.append((work, flat, gs))

    def finish(self):
        if self.mesh.dp == 1:
            return
        if not self._hooked:
            for p in self.model.parameters():
                if p.grad is not None:
                    self._add(p.grad)
        for mod in self.model.modules():
            if isinstance(mod, NVFP4Linear) and mod.no_master and mod.grad_w is not None:
                self._add(mod.grad_w)
        self._launch()
        for work, flat, gs in self._pending:
            work.wait()
            off = 0
            for g in gs:
                n = g.numel()
                g.copy_(flat[off:off + n].view_as(g)); off += n
        self._pending = []
