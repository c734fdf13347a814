#!/usr/bin/env python
"""Training-step probe at 7B width with a reduced layer count: setup_worker + a few train_step calls on one GPU,
printing the phase split (forward/backward, Muon, AdamW), kernel launch count and device status per step.
Small enough to run under `ncu --metrics gpu__time_duration.sum` for a per-kernel share list of one step
(counterpart of the reference's loop step bench, ``test/_tmp/bench_step.py``)."""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from hippolm_b200.cli import build_parser                                  # noqa: E402
from hippolm_b200.train.loop import setup_worker, train_step               # noqa: E402
from hippolm_b200.data.loaders import synthetic_loader                     # noqa: E402
from hippolm_b200.utils.timing import PhaseTimer                           # noqa: E402
from hippolm_b200.ops import _ext                                          # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--seqs", type=int, default=2)
    ap.add_argument("--seq_len", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--bf16_ffn", action="store_true")
    a = ap.parse_args()
    args = build_parser().parse_args([])
    args.vocab_size, args.hidden_size, args.num_heads, args.head_dim = 128256, 4096, 32, 128
    args.num_layers, args.num_blocks, args.intermediate_size = a.layers, max(1, a.layers // 4), 14336
    args.ffn_nvfp4 = args.ffn_nvfp4_no_bf16_master = not a.bf16_ffn
    args.batch_size, args.seq_len, args.micro_batch_size, args.max_steps = a.seqs, a.seq_len, a.seq_len, 10 ** 9
    t0 = time.time()
    loader = synthetic_loader(args.batch_size, args.seq_len, args.vocab_size, 0, a.seq_len, a.seq_len)
    ctx = setup_worker(args, run_dir=None, data_iter=loader)
    torch.cuda.synchronize()
    print("setup s", round(time.time() - t0, 2), flush=True)
    batch = next(loader)
    for i in range(a.steps):
        _ext.reset_launch_count()
        t0 = time.time()
        tm = PhaseTimer(True, ctx.device)
        out = train_step(ctx, batch, tm)
        ctx.step += 1
        torch.cuda.synchronize()
        print(i, "step s", round(time.time() - t0, 3), "loss", round(float(out["loss"]), 4), tm.summary(),
              "launches", _ext.launch_count(), "status", _ext.device_status(), flush=True)
    print("max mem GB", round(torch.cuda.max_memory_allocated() / 2 ** 30, 2))


if __name__ == "__main__":
    main()
