"""GPU selection and process launch (``src/training/launch/gpus.py:7-81``, ``scripts/train.py:126-239``).

``select_gpus`` picks the largest contiguous run of 8/4/2/1 GPUs with enough free memory, reading
free memory through an injectable query (NVML -> torch fallback) so it is testable without a GPU.
``launch`` runs one worker per GPU with ``torch.multiprocessing.spawn`` (or inline when world == 1);
under ``torchrun`` (RANK set) the worker simply runs in this process. Before spawning on a CUDA machine it
picks the GPUs with ``select_gpus(args.min_gpu_memory_mb, want=world)`` and exposes exactly that run to the
workers through ``CUDA_VISIBLE_DEVICES``. ``--tp_sim`` runs the same ranks as CPU processes over gloo
(the reference's TP simulation puts N ranks on one GPU, ``src/training/launch/tp_sim.py:26``; here the
simulated ranks need no GPU at all).

Restart after a failure (``--max_restarts N``, default 0): the workers run as child processes; when any of them ends
with an error (an exception, a lost peer, a watchdog stop, a killed process), ``mp.spawn`` ends the others, and the
launcher starts a new set on a new rendezvous port with ``--resume latest``, so the run continues from the newest
complete checkpoint of its run directory (or from step 0 when none has been written yet). The reference's launcher stops
at the first failure (``scripts/train.py:233-237``).
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
    if os.environ.get("HIPPO_TP_SIM") == "1":
        # simulated ranks share the host's cores: one full-width thread pool per rank would oversubscribe them many times
        import torch
        torch.set_num_threads(max(1, (os.cpu_count() or 1) // max(1, world)))
    fn(args)


def pick_devices(args, world: int, query: Optional[Callable[[], Sequence[int]]] = None,
                 have_cuda: Optional[bool] = None) -> Optional[List[int]]:
    """GPU indices for ``world`` workers, None when the run uses no GPU (CPU box or ``--tp_sim``).
    Raises when fewer than ``world`` contiguous GPUs have ``min_gpu_memory_mb`` free."""
    if bool(getattr(args, "tp_sim", False)):
        return None
    if have_cuda is None:
        import torch
        have_cuda = torch.cuda.is_available()
    if not have_cuda:
        return None
    need = int(getattr(args, "min_gpu_memory_mb", 0) or 0)
    gpus = select_gpus(need, want=world, query=query)
    if len(gpus) != world:
        raise RuntimeError(f"no contiguous run of {world} GPU(s) with {need} MiB free "
                           f"(lower --min_gpu_memory_mb or the number of ranks)")
    return gpus


def launch(fn, args, world: int) -> None:
    if "RANK" in os.environ:
        fn(args)                         # under torchrun: the launcher already chose the devices
        return
    if bool(getattr(args, "tp_sim", False)):
        os.environ["HIPPO_TP_SIM"] = "1"  # ranks become CPU processes over gloo (see parallel/mesh.py)
    gpus = pick_devices(args, max(1, world))
    restarts = max(0, int(getattr(args, "max_restarts", 0) or 0))
    if world <= 1 and restarts == 0:
        if gpus is not None:
            os.environ["LOCAL_RANK"] = str(gpus[0])     # the inline worker binds to the selected GPU
        fn(args)
        return
    world = max(1, world)
    if gpus is not None:
        # the spawned workers see exactly the selected run, as local devices 0..world-1
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        phys = [int(x) for x in vis.split(",")] if vis else None
        os.environ["CUDA_VISIBLE_DEVICES"] = ",".join(str(phys[g] if phys else g) for g in gpus)
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 1000
    attempt = 0
    while True:
        try:
            mp.spawn(_spawn_entry, args=(world, port + attempt, fn, args), nprocs=world, join=True)
            return
        except Exception as ex:                                   # noqa: BLE001  a worker raised, exited or was killed
            if attempt >= restarts:
                raise
            attempt += 1
            import logging
            logging.getLogger("hippo.launch").warning(
                f"worker failure ({type(ex).__name__}: {([l for l in str(ex).splitlines() if l.strip()] or [''])[-1]}); "
                f"restart {attempt} of {restarts} from the latest complete checkpoint")
            args.resume = "latest"
            os.environ["HIPPO_RESTART_ATTEMPT"] = str(attempt)
