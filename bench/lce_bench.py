#!/usr/bin/env python
"""Linear + cross-entropy head of one token chunk, single GPU: fp32 logits with a separate statistics pass against
bf16 logits with the statistics taken in the logits GEMM epilogue (``lce_epilogue_stats``).

    python bench/lce_bench.py [--T 8192 --D 4096 --V 128256]          event timings of both paths, stage by stage
    python bench/lce_bench.py --gemm_ab                               the two logits GEMMs timed alternately (A B A B ...),
                                                                      so that neither runs on a cooler GPU than the other
    python bench/lce_bench.py --profile --T 4096 --V 32064            a few launches of the epilogue-statistics GEMM only
                                                                      (the small case a profiler is pointed at)
"""
import argparse
import json

import torch

from common import time_ms
from hippolm_b200 import ops
from hippolm_b200.ops import cuda_ops as co


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--T", type=int, default=8192)
    ap.add_argument("--D", type=int, default=4096)
    ap.add_argument("--V", type=int, default=128256)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--gemm_ab", action="store_true")
    a = ap.parse_args()
    T, D, V = a.T, a.D, a.V
    torch.manual_seed(0)
    x = torch.randn(T, D, device="cuda").bfloat16()
    w = (0.02 * torch.randn(V, D, device="cuda")).bfloat16()
    tg = torch.randint(0, V, (T,), device="cuda")
    roww = torch.full((T,), 1.0 / T, device="cuda")
    loss = torch.zeros(1, device="cuda")

    if a.profile:
        for _ in range(3):
            co.lce_logits_stats(x, w, tg)
        torch.cuda.synchronize()
        print(json.dumps({"profile_case": {"T": T, "D": D, "V": V}, "launches": 3}))
        return

    flops = 2.0 * T * D * V
    rec = {"T": T, "D": D, "V": V, "iters": a.iters}

    if a.gemm_ab:
        fa, fb = [], []
        for _ in range(4):
            fa.append(round(time_ms(lambda: co.gemm_nt(x, w, out_dtype=torch.float32), warmup=1, iters=3), 3))
            fb.append(round(time_ms(lambda: co.lce_logits_stats(x, w, tg), warmup=1, iters=3), 3))
        fc = round(time_ms(lambda: co.gemm_nt(x, w), warmup=1, iters=3), 3)
        rec.update({"alternating_fp32_out_ms": fa, "alternating_epilogue_stats_ms": fb, "bf16_out_plain_ms": fc,
                    "tflops_fp32_out_last": round(flops / fa[-1] / 1e9, 1),
                    "tflops_epilogue_stats_last": round(flops / fb[-1] / 1e9, 1)})
        print(json.dumps(rec), flush=True)
        return

    # stage by stage
    t = time_ms(lambda: co.gemm_nt(x, w, out_dtype=torch.float32), iters=a.iters)
    rec["logits_gemm_fp32_ms"] = round(t, 3); rec["logits_gemm_fp32_tflops"] = round(flops / t / 1e9, 1)
    t = time_ms(lambda: co.lce_logits_stats(x, w, tg), iters=a.iters)
    rec["logits_gemm_epilogue_stats_ms"] = round(t, 3); rec["logits_gemm_epilogue_stats_tflops"] = round(flops / t / 1e9, 1)
    z32, mx, se, tz = co.lce_chunk_stats(x, w, tg)
    rec["fp32_stats_plus_gemm_ms"] = round(time_ms(lambda: co.lce_chunk_stats(x, w, tg), iters=a.iters), 3)
    lse = mx + se.log()
    rec["fp32_grad_ms"] = round(time_ms(lambda: co.lce_chunk_grad(z32, lse, tg, roww), iters=a.iters), 3)
    del z32
    z, part, tzb, tg64 = co.lce_logits_stats(x, w, tg)
    rec["bf16_merge_plus_grad_inplace_ms"] = round(
        time_ms(lambda: co.lce_grad_inplace_local(z, part, tzb, tg64, roww, loss), iters=a.iters), 3)
    del z, part

    # whole chunk: logits, statistics, gradient, dX and dW GEMMs
    dw = torch.zeros(V, D, dtype=torch.float32, device="cuda")

    def chunk_fp32():
        zc, m_, s_, _t = co.lce_chunk_stats(x, w, tg)
        pz = co.lce_chunk_grad(zc, m_ + s_.log(), tg, roww)
        ops.gemm_nn(pz, w)
        ops.gemm_tn_accumulate(pz, x, dw)

    def chunk_epi():
        zc, p_, t_, g_ = co.lce_logits_stats(x, w, tg)
        pz = co.lce_grad_inplace_local(zc, p_, t_, g_, roww, loss)
        ops.gemm_nn(pz, w)
        ops.gemm_tn_accumulate(pz, x, dw)

    for name, fn in (("chunk_fp32_logits", chunk_fp32), ("chunk_epilogue_stats", chunk_epi)):
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        rec[name + "_ms"] = round(time_ms(fn, iters=a.iters), 3)
        rec[name + "_peak_extra_gb"] = round((torch.cuda.max_memory_allocated() - base) / 2 ** 30, 2)
    rec["chunk_tflops_epilogue_stats"] = round(3 * flops / rec["chunk_epilogue_stats_ms"] / 1e9, 1)
    print(json.dumps(rec))


if __name__ == "__main__":
    main()
