#!/usr/bin/env python
"""Fused all-gather->GEMM / GEMM->reduce-scatter vs NCCL + plain GEMM, device-timed, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench/fused_comm_bench.py

For each shape prints the NCCL collective alone, the GEMM alone, their sum (unfused path), the fused kernel and its
fraction of the roofline max(GEMM at measured peak, NVLink bytes / 770 GB/s)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from hippolm_b200.parallel.mesh import init_distributed_from_env, init_mesh   # noqa: E402
from hippolm_b200.parallel import fused                                        # noqa: E402
from hippolm_b200.parallel.collectives import all_gather_dim0, reduce_scatter_dim0   # noqa: E402
from hippolm_b200.ops import cuda_ops as co, _ext                              # noqa: E402
from hippolm_b200.utils.timing import load_measured_peaks                      # noqa: E402


def timed(fn, group, iters=10):
    for _ in range(3):
        fn()
    dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    dev = init_distributed_from_env()
    w = dist.get_world_size()
    mesh = init_mesh(tp=w, device=dev)
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=0, help="tokens per call; 0 = 8192 per rank (the training micro-batch)")
    ap.add_argument("--comm_ctas", type=int, default=0, help="copy CTAs of the all-gather kernels (0 = the default, 16)")
    a = ap.parse_args()
    T, D = a.tokens or 8192 * w, 4096
    assert fused.setup(mesh, T, D)
    ws = fused._STATE["ws"]
    if a.comm_ctas > 0:
        ws.comm_ctas = a.comm_ctas
    pk = load_measured_peaks()
    g = mesh.tp_group
    for (name, N, K) in [("attn in_proj", 6400 // w // 64 * 64, D), ("ffn gate_up", 2 * 14336 // w, D)]:
        x = torch.randn(T // w, K, device=dev).bfloat16(); W = (0.02 * torch.randn(N, K, device=dev)).bfloat16()
        xg = all_gather_dim0(x, g, w)
        t_ag = timed(lambda: all_gather_dim0(x, g, w), g)
        t_mm = timed(lambda: co.gemm_nt(xg, W), g)
        t_f = timed(lambda: ws.allgather_gemm(x, W, need_gathered=False), g)
        roof = max(2.0 * T * N * K / (pk["bf16_tflops"] * 1e12), (w - 1) * x.numel() * 2 / (pk["nvlink_gbs"] * 1e9)) * 1e3
        if mesh.rank == 0:
            print(json.dumps({"op": "allgather->gemm " + name, "world": w, "T": T, "N": N, "K": K, "nccl_ag_ms": round(t_ag, 3),
                              "gemm_ms": round(t_mm, 3), "unfused_ms": round(t_ag + t_mm, 3), "fused_ms": round(t_f, 3),
                              "roofline_ms": round(roof, 3), "fused_frac_of_roofline": round(roof / t_f, 3)}), flush=True)
    for (name, N, K) in [("attn o_proj", D, 4096 // w), ("ffn down", D, 14336 // w // 8 * 8)]:
        a = torch.randn(T, K, device=dev).bfloat16(); W = (0.02 * torch.randn(N, K, device=dev)).bfloat16()
        y = co.gemm_nt(a, W)
        t_rs = timed(lambda: reduce_scatter_dim0(y, g, w), g)
        t_mm = timed(lambda: co.gemm_nt(a, W), g)
        t_f = timed(lambda: ws.gemm_reduce_scatter(a, W), g)
        roof = max(2.0 * T * N * K / (pk["bf16_tflops"] * 1e12), (w - 1) / w * T * N * 2 / (pk["nvlink_gbs"] * 1e9)) * 1e3
        if mesh.rank == 0:
            print(json.dumps({"op": "gemm->reduce_scatter " + name, "world": w, "T": T, "N": N, "K": K, "nccl_rs_ms": round(t_rs, 3),
                              "gemm_ms": round(t_mm, 3), "unfused_ms": round(t_rs + t_mm, 3), "fused_ms": round(t_f, 3),
                              "roofline_ms": round(roof, 3), "fused_frac_of_roofline": round(roof / t_f, 3)}), flush=True)
    # NVFP4 FFN: quantise-and-push -> FP4 GEMM (0.5625 bytes per element on the wire) and FP4 GEMM -> reduce-scatter.
    # FP4 tensor-core peak is taken as 4x the measured bf16 peak (no measured FP4 figure exists).
    from hippolm_b200.ops import nvfp4_cuda, fp4_gemm
    fp4_peak = 4.0 * pk["bf16_tflops"] * 1e12
    N, K = 2 * 14336 // w, D
    x = torch.randn(T // w, K, device=dev).bfloat16(); W = (0.02 * torch.randn(N, K, device=dev)).bfloat16()
    wp, wsc, wgs = nvfp4_cuda.quantize(W)
    xg = all_gather_dim0(x, g, w)
    t_ag = timed(lambda: all_gather_dim0(x, g, w), g)
    t_mm = timed(lambda: fp4_gemm.gemm_nt(xg, wp, wsc, wgs), g)
    t_f = timed(lambda: ws.nvfp4_allgather_gemm(x, wp, wsc, wgs), g)
    roof = max(2.0 * T * N * K / fp4_peak, (w - 1) * x.numel() * 0.5625 / (pk["nvlink_gbs"] * 1e9)) * 1e3
    if mesh.rank == 0:
        print(json.dumps({"op": "nvfp4 quantise+push->gemm ffn gate_up", "world": w, "T": T, "N": N, "K": K,
                          "nccl_ag_bf16_ms": round(t_ag, 3), "quant+fp4_gemm_ms": round(t_mm, 3),
                          "unfused_ms": round(t_ag + t_mm, 3), "fused_ms": round(t_f, 3), "roofline_ms": round(roof, 3),
                          "fused_frac_of_roofline": round(roof / t_f, 3)}), flush=True)
    N, K = D, 14336 // w // 256 * 256
    a = torch.randn(T, K, device=dev).bfloat16(); W = (0.02 * torch.randn(N, K, device=dev)).bfloat16()
    wp, wsc, wgs = nvfp4_cuda.quantize(W)
    y = fp4_gemm.gemm_nt(a, wp, wsc, wgs)
    t_rs = timed(lambda: reduce_scatter_dim0(y, g, w), g)
    t_mm = timed(lambda: fp4_gemm.gemm_nt(a, wp, wsc, wgs), g)
    t_f = timed(lambda: ws.nvfp4_gemm_reduce_scatter(a, wp, wsc, wgs), g)
    roof = max(2.0 * T * N * K / fp4_peak, (w - 1) / w * T * N * 2 / (pk["nvlink_gbs"] * 1e9)) * 1e3
    if mesh.rank == 0:
        print(json.dumps({"op": "nvfp4 gemm->reduce_scatter ffn down", "world": w, "T": T, "N": N, "K": K,
                          "nccl_rs_ms": round(t_rs, 3), "quant+fp4_gemm_ms": round(t_mm, 3), "unfused_ms": round(t_rs + t_mm, 3),
                          "fused_ms": round(t_f, 3), "roofline_ms": round(roof, 3),
                          "fused_frac_of_roofline": round(roof / t_f, 3)}), flush=True)
    torch.cuda.synchronize()
    ws.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
