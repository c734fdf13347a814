"""GPU selection and process launch (``src/training/launch/gpus.py:7-81``, ``scripts/train.py:126-239``).

``select_gpus`` picks the largest contiguous run of 8/4/2/1 GPUs with enough free memory, reading
free memory through an injectable query (NVML -> torch fallback) so it is testable without a GPU.
``launch`` runs one worker per GPU with ``torch.multiprocessing.spawn`` (or inline when world == 1);
under ``torchrun`` (RANK set) the worker simply runs in this process.
"""
from __future__ import annotations

import os
from typing import Callable, List, Optional, Sequence


def _query_free_mb_nvml() -> Optional[List[int]]:
    try:
        import pynvml
        pynvml.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = [int(x) for x in vis.split(",")] if vis else list(range(pynvml.nvmlDeviceGetCount()))
        out = []
        for i in idx:
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            out.append(int(pynvml.nvmlDeviceGetMemoryInfo(h).free // 2 ** 20))
        return out
    except Exception:
        return None


def _query_free_mb_torch() -> List[int]:
    import torch
    out = []
    for i in range(torch.cuda.device_count()):
        free, _ = torch.cuda.mem_get_info(i)
        out.append(int(free // 2 ** 20))
    return out


def select_gpus(min_memory_mb: int, want: Optional[int] = None,
                query: Optional[Callable[[], Sequence[int]]] = None) -> List[int]:
    """Largest contiguous run (8, 4, 2, then 1 long) of local GPU indices with >= min_memory_mb free."""
    free = list(query()) if query is not None else (_query_free_mb_nvml() or _query_free_mb_torch())
    ok = [f >= min_memory_mb for f in free]
    sizes = [want] if want else [8, 4, 2, 1]
    for n in sizes:
        for s in range(0, len(ok) - n + 1):
            if all(ok[s:s + n]):
                return list(range(s, s + n))
    return []


def _spawn_entry(rank: int, world: int, port: int, fn, args):
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    fn(args)


def launch(fn, args, world: int) -> None:
    if "RANK" in os.environ or world <= 1:
        fn(args)
        return
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 1000
    mp.spawn(_spawn_entry, args=(world, port, fn, args), nprocs=world, join=True)
