"""Timing and roofline helpers.

``PhaseTimer`` reproduces the reference's ``--mb_timing`` host phase split
(``src/training/loop/run.py:125-528``); ``DeviceTimer`` is the CUDA-event timer used for every
reported number (max over ranks is taken by the caller); ``roofline`` turns a measured time into a
fraction of the slower of compute-at-peak and bytes-over-the-link.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from typing import Dict, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """Host phase split of one step (synchronised at the phase borders on a GPU). With ``events`` (a list shared by the
    steps of a run) every phase occurrence is also recorded as ``(name, start in us since the epoch, duration in us,
    step)`` for ``write_chrome_trace``."""

    def __init__(self, enabled: bool = True, device: Optional[torch.device] = None, events: Optional[list] = None,
                 step: int = 0, memory=None):
        self.enabled = enabled
        self.memory = memory                   # a ``utils.vram.PhaseMemory``: peak device memory inside every phase
        self.cuda = device is not None and device.type == "cuda"
        self.ms: Dict[str, float] = {}
        self.events, self.step = events, step

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            with nvtx_range(name):
                yield
            return
        if self.cuda:
            torch.cuda.synchronize()
        if self.memory is not None:
            self.memory.begin()
        t0 = time.perf_counter()
        with nvtx_range(name):
            yield
        if self.cuda:
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if self.memory is not None:
            self.memory.record(name, self.step)
        self.ms[name] = self.ms.get(name, 0.0) + dt * 1e3
        if self.events is not None:
            self.events.append((name, (time.time() - dt) * 1e6, dt * 1e6, self.step))

    def summary(self) -> Dict[str, float]:
        return {k: round(v, 3) for k, v in self.ms.items()}


def write_chrome_trace(path: str, events, rank: int = 0) -> None:
    """Phase occurrences recorded by ``PhaseTimer`` as a Chrome / Perfetto trace (``chrome://tracing``, ui.perfetto.dev):
    one complete event per phase occurrence, process = rank, the step number in ``args``."""
    out = [{"name": n, "ph": "X", "ts": ts, "dur": dur, "pid": rank, "tid": 0, "args": {"step": step}}
           for (n, ts, dur, step) in events]
    out.append({"name": "process_name", "ph": "M", "pid": rank, "args": {"name": f"rank {rank}"}})
    with open(path, "w") as f:
        json.dump({"traceEvents": out, "displayTimeUnit": "ms"}, f)


class DeviceTimer:
    """CUDA events on the current stream; ``elapsed_ms`` synchronises."""

    def __init__(self):
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e1 = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        self.e0.record()
        return self

    def __exit__(self, *a):
        self.e1.record()

    def elapsed_ms(self) -> float:
        self.e1.synchronize()
        return self.e0.elapsed_time(self.e1)


def load_measured_peaks(repo_root: Optional[str] = None) -> Dict[str, float]:
    """Measured denominators when the driver-written file is present, else the stated fallback."""
    root = repo_root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "nvlink_gbs": 770.0, "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "nvlink_gbs": 770.0, "source": "fallback"}


def roofline(ms: float, flops: float = 0.0, hbm_bytes: float = 0.0, link_bytes: float = 0.0,
             peaks: Optional[Dict[str, float]] = None, sustained: bool = False) -> Dict[str, float]:
    """achieved / roofline where roofline time = max(flops/peak, hbm bytes/bw, link bytes/link bw)."""
    pk = peaks or load_measured_peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
    t_c = flops / tf if flops else 0.0
    t_m = hbm_bytes / (pk["hbm_gbs"] * 1e9) if hbm_bytes else 0.0
    t_l = link_bytes / (pk["nvlink_gbs"] * 1e9) if link_bytes else 0.0
    t_roof = max(t_c, t_m, t_l)
    return {"roofline_ms": t_roof * 1e3, "fraction": (t_roof * 1e3 / ms) if ms > 0 else 0.0,
            "bound": "compute" if t_roof == t_c else ("hbm" if t_roof == t_m else "nvlink"),
            "peaks": pk["source"]}
