#!/usr/bin/env python
"""Throughput of the host-side fused accumulator / optimizer kernels (``csrc/host_fused.cpp``) on 32 M elements:
wall-clock median of 5 calls, bytes = every element read or written once. ``HIPPO_HOST_ISA=avx2`` times the AVX2 build,
``HIPPO_FUSED_FORCE_PYLOOP=1`` the torch fallback. Runs on the CPU alone."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from hippolm_b200.optim import host_fused as hf  # noqa: E402

torch.manual_seed(0)
n = 1 << 25


def bench(name, fn, nbytes, reps=5):
    fn()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter(); fn(); ts.append(time.perf_counter() - t0)
    t = sorted(ts)[len(ts) // 2]
    print(f"{name:32s} {t * 1e3:8.2f} ms  {nbytes / t / 1e9:7.1f} GB/s")


print(f"host kernels: {hf.isa()}, {torch.get_num_threads()} torch threads")
for dt in (torch.bfloat16, torch.float32):
    a = torch.randn(n).to(dt); b = torch.randn(n).to(dt); es = a.element_size()
    bench(f"add_into_many {dt}", lambda: hf.fused_add_into_many([a], [b]), 3 * n * es)
    bench(f"scale_many {dt}", lambda: hf.fused_scale_many([a], 0.999), 2 * n * es)
    bench(f"l2_norm_sq {dt}", lambda: hf.fused_l2_norm_sq([a]), n * es)
    bench(f"inf_nan_count {dt}", lambda: hf.fused_inf_nan_count([a]), n * es)
    g = torch.randn(n).to(dt); m = torch.zeros(n).to(dt); v = torch.zeros(n).to(dt)
    bench(f"adam_step {dt}", lambda: hf.fused_adam_step(g, m, v, 0.9, 0.95, 1e-8, 3), 6 * n * es)
