"""Process mesh: world = dp x tp, one process per GPU.

TP ranks are contiguous (rank = dp_rank * tp + tp_rank) so a TP group sits on NVSwitch
neighbours. The reference only has a single TP group that is the whole world
(``src/models/tp_model/_primitives.py:53-132``); data parallelism is new here.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class Mesh:
    world_size: int = 1
    rank: int = 0
    tp: int = 1
    dp: int = 1
    tp_rank: int = 0
    dp_rank: int = 0
    tp_group: Optional[object] = None
    dp_group: Optional[object] = None
    device: torch.device = torch.device("cpu")

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1

    def tp_ranks(self):
        base = self.dp_rank * self.tp
        return list(range(base, base + self.tp))

    def dp_ranks(self):
        return [d * self.tp + self.tp_rank for d in range(self.dp)]


_MESH = Mesh()


def get_mesh() -> Mesh:
    return _MESH


def init_mesh(tp: int = 1, dp: Optional[int] = None, device: Optional[torch.device] = None) -> Mesh:
    """Build TP and DP groups on top of an initialised default process group (or none)."""
    global _MESH
    if dist.is_available() and dist.is_initialized():
        world, rank = dist.get_world_size(), dist.get_rank()
    else:
        world, rank = 1, 0
    if dp is None:
        assert world % tp == 0, f"world {world} not divisible by tp {tp}"
        dp = world // tp
    assert tp * dp == world, f"tp({tp}) x dp({dp}) != world({world})"
    m = Mesh(world_size=world, rank=rank, tp=tp, dp=dp, tp_rank=rank % tp, dp_rank=rank // tp,
             device=device if device is not None else torch.device("cpu"))
    if world > 1:
        # every rank must create every group, in the same order
        for d in range(dp):
            ranks = list(range(d * tp, (d + 1) * tp))
            g = dist.new_group(ranks) if tp > 1 else None
            if d == m.dp_rank:
                m.tp_group = g
        for t in range(tp):
            ranks = [d * tp + t for d in range(dp)]
            g = dist.new_group(ranks) if dp > 1 else None
            if t == m.tp_rank:
                m.dp_group = g
    _MESH = m
    return m


def reset_mesh() -> None:
    global _MESH
    _MESH = Mesh()


def init_distributed_from_env(backend: Optional[str] = None, timeout_s: float = 1800.0) -> torch.device:
    """env:// rendezvous (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT)."""
    import datetime
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    # HIPPO_TP_SIM=1 (``--tp_sim``): simulated ranks are CPU processes over gloo even on a GPU machine
    use_cuda = torch.cuda.is_available() and os.environ.get("HIPPO_TP_SIM", "0") != "1"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        backend = backend or ("nccl" if use_cuda else "gloo")
        kw = {}
        if backend == "nccl":
            kw["device_id"] = device
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return device
