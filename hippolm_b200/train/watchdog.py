"""Host-side step watchdog + heartbeat file.

Failure detection stays on the host: a daemon thread checks that ``beat(step)`` keeps arriving;
when the gap exceeds the timeout it records the stall (log + ``heartbeat.rank{r}.json``) and runs the
``on_stall`` callback (default: nothing; the launcher can decide to restart from the latest
checkpoint). Device kernels never spin without a bound, so a stall here means a host/peer problem.
"""
from __future__ import annotations

import json
import os
import threading
import time
from typing import Callable, Optional


class StepWatchdog:
    def __init__(self, timeout_s: float, run_dir: Optional[str] = None, rank: int = 0,
                 on_stall: Optional[Callable[[int, float], None]] = None, poll_s: float = 0.05):
        self.timeout_s, self.run_dir, self.rank, self.on_stall = timeout_s, run_dir, rank, on_stall
        self.poll_s = poll_s
        self._last = time.monotonic()
        self._step = -1
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.stalled = False

    def start(self):
        self._last = time.monotonic()
        self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)
        self._thread.start()

    def beat(self, step: int):
        self._last = time.monotonic()
        self._step = step
        self.stalled = False
        if self.run_dir:
            try:
                p = os.path.join(self.run_dir, f"heartbeat.rank{self.rank}.json")
                with open(p + ".tmp", "w") as f:
                    json.dump({"step": step, "time": time.time()}, f)
                os.replace(p + ".tmp", p)
            except OSError:
                pass

    def _run(self):
        while not self._stop.wait(self.poll_s):
            gap = time.monotonic() - self._last
            if gap > self.timeout_s and not self.stalled:
                self.stalled = True
                if self.on_stall is not None:
                    self.on_stall(self._step, gap)

    def close(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
