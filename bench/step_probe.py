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
    ap.add_argument("--ffn_bwd", type=str, default="fp4", choices=["bf16", "fp4_dx", "fp4"],
                    help="backward of the NVFP4 FFN linears (the benchmark configuration uses fp4)")
    ap.add_argument("--heads", type=int, default=32, help="e.g. 4 = the local heads of one TP=8 rank")
    ap.add_argument("--ffn", type=int, default=14336, help="e.g. 1792 = the local FFN width of one TP=8 rank")
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--micro", type=int, default=0, help="micro-batch tokens (default: one sequence)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree; > 1 runs under torch.distributed.run with "
                    "that many ranks (full model dimensions, rank 0 prints)")
    ap.add_argument("--no_fused_comm", action="store_true")
    ap.add_argument("--gemm_log", action="store_true", help="time every bf16 GEMM call of one extra step with CUDA events "
                    "and print time and TFLOP/s per (layout, M, N, K) (diagnosis only)")
    ap.add_argument("--kineto", action="store_true", help="after the timed steps, trace one more step with torch.profiler "
                    "and print GPU-busy time vs wall time and the top kernels (diagnosis only, not a benchmark number)")
    a = ap.parse_args()
    args = build_parser().parse_args([])
    args.vocab_size, args.hidden_size, args.num_heads, args.head_dim = a.vocab, 4096, a.heads, 128
    args.num_layers, args.num_blocks, args.intermediate_size = a.layers, max(1, a.layers // 4), a.ffn
    args.attn_res_heads = 32
    args.ffn_nvfp4 = args.ffn_nvfp4_no_bf16_master = not a.bf16_ffn
    args.ffn_nvfp4_backward = "bf16" if a.bf16_ffn else a.ffn_bwd
    args.batch_size, args.seq_len, args.micro_batch_size, args.max_steps = a.seqs, a.seq_len, a.micro or a.seq_len, 10 ** 9
    args.tp_size, args.dp_size, args.fused_comm = a.tp, 1, not a.no_fused_comm
    rank0 = int(os.environ.get("RANK", "0")) == 0
    if not rank0:
        sys.stdout = open(os.devnull, "w")
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
    if a.gemm_log:
        from hippolm_b200.ops import cuda_ops
        orig, recs = cuda_ops._gemm, []

        def timed(a_, b_, layout, M, N, K, *args_, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = orig(a_, b_, layout, M, N, K, *args_, **kw)
            e1.record()
            recs.append(((layout, M, N, K), e0, e1))
            return out
        cuda_ops._gemm = timed
        train_step(ctx, batch)
        torch.cuda.synchronize()
        cuda_ops._gemm = orig
        agg = {}
        for key, e0, e1 in recs:
            c = agg.setdefault(key, [0, 0.0]); c[0] += 1; c[1] += e0.elapsed_time(e1)
        tot = sum(v[1] for v in agg.values())
        print(f"bf16 GEMM calls {len(recs)}, total {tot:.1f} ms")
        for (layout, M, N, K), (c, ms) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:40]:
            tf = 2.0 * M * N * K * c / ms / 1e9
            print(f"  {ms:8.2f} ms {c:5d} x  {'NT NN TN TT'.split()[layout]} M={M:6d} N={N:6d} K={K:6d}  {tf:7.1f} TFLOP/s")
    if a.kineto:
        from torch.profiler import profile, ProfilerActivity
        torch.cuda.synchronize()
        t0 = time.time()
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True) as prof:
            train_step(ctx, batch)
            torch.cuda.synchronize()
        wall = time.time() - t0
        ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
        busy = sum(e.device_time for e in ev) / 1e3
        print(f"traced step: wall {wall * 1e3:.1f} ms, sum of GPU kernel time {busy:.1f} ms, kernels {len(ev)}")
        agg = {}
        for e in ev:
            k = e.name.split("<")[0].split("(")[0][:60]
            c = agg.setdefault(k, [0, 0.0]); c[0] += 1; c[1] += e.device_time / 1e3
        for k, (c, ms) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:25]:
            print(f"  {ms:9.2f} ms {c:6d}  {k}")
        # library (aten) operators by their own GPU time, with input shapes: what is left of torch glue in the step
        print("aten operators by self GPU time:")
        ops = [e for e in prof.key_averages(group_by_input_shape=True) if e.key.startswith("aten::") and e.self_device_time_total > 0]
        for e in sorted(ops, key=lambda e: -e.self_device_time_total)[:30]:
            print(f"  {e.self_device_time_total / 1e3:9.2f} ms {e.count:6d}  {e.key}  {str(e.input_shapes)[:110]}")


if __name__ == "__main__":
    main()
