"""VRAM tooling (``tools/vram_profile/*.py``): memory-history snapshots, a polling thread on
``torch.cuda.mem_get_info`` and a saved-tensor size probe."""
from __future__ import annotations

import contextlib
import threading
import time
from typing import Dict, List, Optional

import torch


@contextlib.contextmanager
def memory_history(snapshot_path: Optional[str] = None, max_entries: int = 100000):
    """Records allocator history for the block and optionally dumps a snapshot file for pytorch.org/memory_viz."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.memory._record_memory_history(max_entries=max_entries)
    try:
        yield
    finally:
        if on:
            if snapshot_path:
                torch.cuda.memory._dump_snapshot(snapshot_path)
            torch.cuda.memory._record_memory_history(enabled=None)


class VramPoller:
    """Samples used device memory every ``period_s`` (100 Hz by default) on a daemon thread."""

    def __init__(self, device: int = 0, period_s: float = 0.01):
        self.device, self.period_s = device, period_s
        self.samples: List[float] = []
        self._stop = threading.Event()
        self._t: Optional[threading.Thread] = None

    def start(self):
        def run():
            while not self._stop.wait(self.period_s):
                free, total = torch.cuda.mem_get_info(self.device)
                self.samples.append((total - free) / 2 ** 20)
        self._t = threading.Thread(target=run, name="vram-poller", daemon=True)
        self._t.start()
        return self

    def stop(self) -> Dict[str, float]:
        self._stop.set()
        if self._t:
            self._t.join(timeout=1.0)
        s = self.samples or [0.0]
        return {"peak_mb": max(s), "mean_mb": sum(s) / len(s), "samples": len(s)}


class SavedTensorProbe:
    """Sums the bytes autograd saves for backward inside the block (``saved_tensors_hooks``)."""

    def __init__(self):
        self.bytes = 0
        self.count = 0
        self._seen = set()

    def __enter__(self):
        def pack(t):
            key = (t.data_ptr(), t.numel())
            if key not in self._seen:
                self._seen.add(key)
                self.bytes += t.numel() * t.element_size(); self.count += 1
            return t
        self._ctx = torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t)
        self._ctx.__enter__()
        return self

    def __exit__(self, *a):
        return self._ctx.__exit__(*a)


def vram_line(device) -> str:
    if not torch.cuda.is_available():
        return "vram n/a"
    return (f"vram alloc {torch.cuda.memory_allocated(device) / 2**20:.0f} MiB reserved "
            f"{torch.cuda.memory_reserved(device) / 2**20:.0f} MiB max {torch.cuda.max_memory_allocated(device) / 2**20:.0f} MiB")
