"""Gradient host offload: pinned accumulators, async D2H copies, a host add worker thread.

Every parameter (and every no-master NVFP4 module) gets a pinned host accumulator. A
post-accumulate-grad hook copies the finished gradient to a pinned staging buffer on a dedicated
copy stream, records an event, hands ``(event, accumulator, staging)`` to the ``cpu-add-worker``
thread and frees ``p.grad``; the worker waits for the event and adds with the host C++ kernels.
Before the optimizer step ``drain_to_device`` waits for the queue and uploads the accumulated
gradients. Same moving parts as ``src/training/param_offload/offload.py:133-857`` (hooks, worker,
drain with timeout and synchronous fallback), minus the CPU-resident optimizer, which is optional here.
"""
from __future__ import annotations

import queue
import threading
import time
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..models.nvfp4_linear import NVFP4Linear
from . import host_fused


def _pin(t: torch.Tensor) -> torch.Tensor:
    if torch.cuda.is_available():
        try:
            return t.pin_memory()
        except Exception:
            return t
    return t


class GradOffloader:
    def __init__(self, model: nn.Module, device: torch.device, accum_dtype=torch.bfloat16, async_worker: bool = True,
                 manual_flush: Optional[List[nn.Parameter]] = None):
        self.model, self.device = model, device
        self.cuda = device.type == "cuda"
        self.accum: Dict[int, torch.Tensor] = {}
        self.owner: Dict[int, object] = {}
        self.manual = {id(p) for p in (manual_flush or [])}
        self.copy_stream = torch.cuda.Stream(device) if self.cuda else None
        self._q: "queue.Queue" = queue.Queue()
        self._inflight = 0
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._err: Optional[BaseException] = None
        self._worker: Optional[threading.Thread] = None
        self.handles = []
        for p in model.parameters():
            if p.requires_grad:
                self.accum[id(p)] = _pin(torch.zeros(p.shape, dtype=accum_dtype))
                self.owner[id(p)] = p
                if id(p) not in self.manual:
                    self.handles.append(p.register_post_accumulate_grad_hook(self._hook))
        for mod in model.modules():
            if isinstance(mod, NVFP4Linear) and mod.no_master:
                self.accum[id(mod)] = _pin(torch.zeros((mod.out_features, mod.in_features), dtype=accum_dtype))
                self.owner[id(mod)] = mod
                mod.grad_sink = self._nvfp4_sink
        if async_worker:
            self._start_worker()

    # ------------------------------------------------------------------ worker
    def _start_worker(self):
        self._worker = threading.Thread(target=self._run, name="cpu-add-worker", daemon=True)
        self._worker.start()

    def _run(self):
        while not self._stop.is_set():
            try:
                item = self._q.get(timeout=0.05)
            except queue.Empty:
                continue
            batch = [item]
            while len(batch) < 32:
                try:
                    batch.append(self._q.get_nowait())
                except queue.Empty:
                    break
            try:
                for ev, _, _ in batch:
                    if ev is not None:
                        ev.synchronize()
                host_fused.fused_add_into_many([b[1] for b in batch], [b[2] for b in batch])
            except BaseException as ex:      # surfaced by drain()
                self._err = ex
            finally:
                with self._lock:
                    self._inflight -= len(batch)

    def _enqueue(self, key: int, g: torch.Tensor):
        acc = self.accum[key]
        if self.cuda:
            self.copy_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.copy_stream):
                stage = _pin(torch.empty(g.shape, dtype=acc.dtype))
                stage.copy_(g.to(acc.dtype), non_blocking=True)
                g.record_stream(self.copy_stream)
                ev = torch.cuda.Event()
                ev.record(self.copy_stream)
        else:
            stage, ev = g.detach().to(acc.dtype).clone(), None
        if self._worker is None:
            if ev is not None:
                ev.synchronize()
            host_fused.fused_add_into_many([acc], [stage])
            return
        with self._lock:
            self._inflight += 1
        self._q.put((ev, acc, stage))

    def _hook(self, p: nn.Parameter):
        if p.grad is None:
            return
        self._enqueue(id(p), p.grad)
        p.grad = None

    def _nvfp4_sink(self, mod: NVFP4Linear, dw: torch.Tensor):
        self._enqueue(id(mod), dw)

    # ------------------------------------------------------------------ loop-facing API
    def flush_manual(self):
        """Parameters whose gradient has several producers (a tied embedding) are flushed once per micro-batch."""
        for key in self.manual:
            p = self.owner[key]
            if p.grad is not None:
                self._enqueue(key, p.grad)
                p.grad = None

    def after_microbatch(self):
        self.flush_manual()

    def drain(self, timeout_s: float = 60.0) -> bool:
        """Wait until the worker has consumed everything. Returns False on timeout (the caller may fall back
        to the synchronous path); re-raises a worker exception."""
        t0 = time.monotonic()
        while True:
            with self._lock:
                n = self._inflight
            if n == 0:
                break
            if time.monotonic() - t0 > timeout_s:
                return False
            time.sleep(0.0005)
        if self._err is not None:
            err, self._err = self._err, None
            raise RuntimeError("cpu-add-worker failed") from err
        return True

    def host_grads(self) -> List[torch.Tensor]:
        return list(self.accum.values())

    def grad_norm_sq(self) -> float:
        return host_fused.fused_l2_norm_sq(self.host_grads())

    def inf_nan_count(self) -> int:
        return host_fused.fused_inf_nan_count(self.host_grads())

    def scale(self, coef: float):
        host_fused.fused_scale_many(self.host_grads(), coef)

    def zero(self):
        host_fused.fused_zero_many(self.host_grads())

    def drain_to_device(self, timeout_s: float = 60.0):
        """Upload the accumulated gradients as ``p.grad`` / ``module.grad_w`` and clear the host accumulators."""
        if not self.drain(timeout_s):
            raise TimeoutError("gradient offload queue did not drain")
        for key, acc in self.accum.items():
            own = self.owner[key]
            g = acc.to(self.device, non_blocking=True) if self.cuda else acc.clone()
            if isinstance(own, NVFP4Linear):
                own.grad_w = g
            else:
                own.grad = g.to(own.dtype)
        if self.cuda:
            torch.cuda.current_stream(self.device).synchronize()
        self.zero()

    def close(self):
        try:
            self.drain(5.0)
        except Exception:
            pass
        self._stop.set()
        if self._worker is not None:
            self._worker.join(timeout=2.0)
            self._worker = None
        for h in self.handles:
            h.remove()
        self.handles = []
        for own in self.owner.values():
            if isinstance(own, NVFP4Linear):
                own.grad_sink = None
