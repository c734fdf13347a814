"""Timing helpers for the per-kernel benches: CUDA events on the launching stream, warm-up, an L2 flush
(a write larger than the 126 MB L2) between timed iterations, median over iterations."""
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def time_ms(fn, warmup: int = 3, iters: int = 10, flush: bool = True) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)
