#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the ~7B hybrid KDA/attention decoder.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference ...                      (reference arm)

Model/config: 32 layers at 3:1 KDA:attention, d_model 4096, 32 heads x 128, FFN 14336 (NVFP4, no
bf16 master, forward and backward on the FP4 tensor cores; --ffn_bwd bf16 for the A/B), vocab 128256,
block attention residuals (8 blocks), Muon + AdamW, seq 8192,
TP = N with sequence parallelism. Weak scaling: 16 sequences per GPU per step (N=8 gives the
configured global batch of 128). Synthetic seeded uniform-random tokens, random-init weights.

Timing: W untimed steps, then K steps between barrier + synchronize, CUDA events on the launching
stream, max over ranks. A second K-step loop measures the same metric end to end through the public
``train_step`` API with the per-step D2H read of the loss. Weights (>9 GB/GPU) and activations exceed
the 126 MB L2, so no explicit flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

SEQS_PER_GPU = 16
SEQ_LEN = 8192


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours")
    p.add_argument("--model", type=str, default="7b", help="7b | 1p3b | tiny (tiny/1p3b are for smoke runs only)")
    p.add_argument("--micro_batch_tokens", type=int, default=0,
                   help="tokens per micro-batch; 0 = 8192 x number of GPUs (activations per rank stay constant under TP + SP)")
    p.add_argument("--seqs_per_gpu", type=int, default=SEQS_PER_GPU)
    p.add_argument("--no_fused_comm", action="store_true")
    p.add_argument("--bf16_ffn", action="store_true")
    p.add_argument("--ffn_bwd", type=str, default="fp4",
                   help="NVFP4 FFN backward: fp4 (dX and dW on the FP4 tensor cores, the benchmarked configuration: "
                        "configs/hybrid_7b_tp8.yml) | fp4_dx | bf16 (backward on the dequantised weight; A/B switch)")
    p.add_argument("--lce_epilogue", type=int, default=-1,
                   help="softmax statistics of the loss head in the logits GEMM epilogue (bf16 logits): 1 | 0 | -1 = the "
                        "benchmarked default (on; 0 = fp32 logits and a separate statistics pass, the A/B switch)")
    p.add_argument("--no_kda", dest="kda", action="store_false",
                   help="skip the standalone chunked-KDA timing that rank 0 adds to the JSON line (outside the timed region)")
    p.add_argument("--kda_only", action="store_true", help="print only the standalone chunked-KDA timing")
    p.add_argument("--ref_ffn", type=str, default="nvfp4", help="reference arm FFN storage: nvfp4 (dequantise + cuBLAS) | bf16")
    p.add_argument("--ref_budget_s", type=float, default=1500.0,
                   help="reference arm: wall-clock budget; fewer than --steps steps are timed if they would not fit")
    return p.parse_args()


MODELS = {
    "7b": dict(vocab_size=128256, hidden_size=4096, num_heads=32, head_dim=128, num_layers=32, num_blocks=8,
               intermediate_size=14336, name="hybrid-kda-7b (32L 3:1 KDA:attn, d4096, 32x128, ffn14336 nvfp4, v128256)"),
    "1p3b": dict(vocab_size=128256, hidden_size=2048, num_heads=16, head_dim=128, num_layers=24, num_blocks=6,
                 intermediate_size=5632, name="hybrid-kda-1.3b"),
    "tiny": dict(vocab_size=8192, hidden_size=512, num_heads=4, head_dim=128, num_layers=4, num_blocks=2,
                 intermediate_size=1024, name="hybrid-kda-tiny"),
}


def kda_times(B=4, T=8192, H=16, D=128, docs=8, iters=10):
    """Standalone chunked-KDA forward and forward+backward time through the public autograd op (B=4, T=8192, H=16,
    K=V=128, 8 documents, bf16), CUDA events, warm-up, L2 flushed between iterations."""
    import statistics
    import torch
    import torch.nn.functional as F
    from hippolm_b200.ops.kda_cuda import _KDAFunction
    torch.manual_seed(0)
    dev, TT = "cuda", B * T
    q = F.normalize(torch.randn(TT, H, D, device=dev), dim=-1).bfloat16().requires_grad_(True)
    k = F.normalize(torch.randn(TT, H, D, device=dev), dim=-1).bfloat16().requires_grad_(True)
    v = torch.randn(TT, H, D, device=dev).bfloat16().requires_grad_(True)
    g = (-F.softplus(torch.randn(TT, H, D, device=dev))).requires_grad_(True)
    beta = torch.sigmoid(torch.randn(TT, H, device=dev)).requires_grad_(True)
    h0 = torch.zeros(docs, H, D, D, device=dev)
    cuts = torch.sort(torch.randperm(TT - 1)[:docs - 1] + 1).values
    cu = torch.cat([torch.zeros(1, dtype=torch.long), cuts, torch.tensor([TT])]).to(torch.int32).to(dev)
    do = torch.randn(TT, H, D, device=dev).bfloat16()
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev)

    def fwd():
        with torch.no_grad():
            _KDAFunction.apply(q, k, v, g, beta, h0, cu)

    def fwd_bwd():
        for t in (q, k, v, g, beta):
            t.grad = None
        o = _KDAFunction.apply(q, k, v, g, beta, h0, cu)
        o = o[0] if isinstance(o, (tuple, list)) else o
        o.backward(do)

    def time_ms(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record(); e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    return {"kda_fwd_ms": round(time_ms(fwd), 3), "kda_fwd_bwd_ms": round(time_ms(fwd_bwd), 3),
            "kda_config": {"B": B, "T": T, "H": H, "K": D, "V": D, "docs": docs, "dtype": "bf16",
                           "l2": "flushed between iterations", "impl": "hippolm_b200 chunked KDA (CUDA)"}}


def main():
    a = parse()
    if a.impl == "reference":
        # the reference arm imports nothing of this repository's package: only baseline/reference_arm.py and the
        # unmodified reference tree under baseline/_ref
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm
        return reference_arm.run_kda_only() if a.kda_only else reference_arm.run_train(a)
    sys.path.insert(0, ROOT)
    sys.path.insert(1, os.path.join(ROOT, "bench"))
    from clocks import ClockSampler
    if a.kda_only:
        print(json.dumps(dict(kda_times(), impl="ours")), flush=True)
        return 0
    import torch
    import torch.distributed as dist
    from hippolm_b200.cli import build_parser
    from hippolm_b200.train.loop import setup_worker, train_step, teardown_worker
    from hippolm_b200.data.loaders import synthetic_loader
    from hippolm_b200.ops import _ext

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if a.gpus != world:
        if a.gpus == 1 and world == 1:
            pass
        elif world == 1 and a.gpus > 1:
            # self-launch one rank per GPU
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.abspath(__file__)] + sys.argv[1:]
            return subprocess.call(cmd)
    if a.micro_batch_tokens <= 0:
        # one 8192-token sequence per GPU and micro-batch: activations per rank stay constant under TP + sequence
        # parallelism, and the per-head KDA state recurrences get `world` sequences to run side by side
        a.micro_batch_tokens = 8192 * world
    m = dict(MODELS[a.model])
    name = m.pop("name")
    args = build_parser().parse_args([])
    for k, v in m.items():
        setattr(args, k, v)
    args.ffn_nvfp4 = not a.bf16_ffn
    args.ffn_nvfp4_no_bf16_master = not a.bf16_ffn
    args.ffn_nvfp4_backward = a.ffn_bwd if not a.bf16_ffn else "bf16"
    args.tp_size = world
    args.dp_size = 1
    args.seq_len = SEQ_LEN if a.model != "tiny" else 1024
    args.batch_size = a.seqs_per_gpu * world
    args.micro_batch_size = a.micro_batch_tokens
    args.max_steps = 10 ** 9
    args.lr_decay_steps = 0
    args.lr_warmup_steps = 200          # WSD warm-up keeps the first steps stable on random-init weights
    args.precision = None
    args.fused_comm = not a.no_fused_comm
    args.lce_epilogue_stats = (a.lce_epilogue != 0)
    args.seed = 0
    gb_tokens = args.batch_size * args.seq_len
    loader = synthetic_loader(args.batch_size, args.seq_len, args.vocab_size, seed=0,
                              doc_len_min=args.seq_len, doc_len_max=args.seq_len)
    ctx = setup_worker(args, run_dir=None, data_iter=loader)
    dev = ctx.device
    batches = [next(loader) for _ in range(2)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(a.warmup):
        out = train_step(ctx, batches[i % 2]); ctx.step += 1
    barrier()
    st = _ext.device_status()
    if st[0] != 0:
        raise RuntimeError(f"device status after warm-up: {st}")

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    # ---- device-timed loop
    _ext.reset_launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        out = train_step(ctx, batches[i % 2]); ctx.step += 1
    e1.record()
    barrier()
    launches = _ext.launch_count()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms) / a.steps
    # ---- end-to-end loop: same public API, loss read back to the host every step
    barrier()
    t0 = time.perf_counter()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last_loss = None
    for i in range(a.steps):
        out = train_step(ctx, batches[i % 2]); ctx.step += 1
        last_loss = float(out["loss"])                      # D2H of the step result
    f1.record()
    barrier()
    wall = time.perf_counter() - t0
    ems = torch.tensor([max(f0.elapsed_time(f1), wall * 1e3)], device=dev)
    if world > 1:
        dist.all_reduce(ems, op=dist.ReduceOp.MAX)
    e2e_ms_step = float(ems) / a.steps
    clocks = sampler.stop() if rank == 0 else None
    h2d = sum(t.numel() * t.element_size() for t in (batches[0]["input_ids"], batches[0]["labels"],
                                                     batches[0]["cu_seqlens"]))
    st = _ext.device_status()
    kda = {}
    if a.kda:
        # second half of the headline metric: standalone chunked-KDA forward+backward (rank 0 only, outside the timed
        # regions; the other ranks wait at the barrier)
        if rank == 0:
            try:
                kda = kda_times()
            except Exception as ex:                                   # noqa: BLE001
                kda = {"kda_unavailable": f"{type(ex).__name__}: {str(ex)[:200]}"}
        barrier()
    if rank == 0:
        rec = {"metric": "train tokens/sec (device-timed, max over ranks)", "value": gb_tokens / (ms_step / 1e3),
               "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_step,
               "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": ("bf16 (FFN weights NVFP4; FFN GEMMs on the FP4 tensor cores forward"
                         + (" and backward)" if a.ffn_bwd == "fp4" else ", dX too)" if a.ffn_bwd == "fp4_dx" else ")"))
               if not a.bf16_ffn else "bf16", "data": "synthetic seeded uniform-random tokens, random-init weights",
               "config": {"model": name, "global_batch": args.batch_size, "seq_len": args.seq_len,
                          "parallelism": f"tp{world}+sp", "micro_batch_tokens": a.micro_batch_tokens,
                          "optimizer": "muon+adamw", "l2": "inputs larger than L2 (no explicit flush)",
                          "fused_comm": bool(ctx.extras.get("fused_comm", False)), "ffn_backward": a.ffn_bwd,
                          "lce_epilogue_stats": bool(args.lce_epilogue_stats)},
               "clocks": clocks,
               "e2e": {"value": gb_tokens / (e2e_ms_step / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms_step},
               "gpu_launches": launches, "loss": last_loss,
               "max_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1), "device_status": list(st), "impl": "ours"}
        try:
            from hippolm_b200.parallel import fused as _fused
            # per (op, shape): did the one-kernel compute+collective path win the timing against NCCL + plain GEMM?
            rec["config"]["fused_comm_choices"] = {"/".join(str(x) for x in k): ("fused" if v else "nccl+gemm")
                                                   for k, v in _fused.choices().items()}
        except Exception:                                              # noqa: BLE001
            pass
        rec.update(kda)
        print(json.dumps(rec), flush=True)
    teardown_worker(ctx)
    return 0


if __name__ == "__main__":
    sys.exit(main())
