#!/usr/bin/env python
"""tcgen05 bf16 GEMM (NT / NN / TN) and block-scaled NVFP4 GEMM throughput against torch.matmul (cuBLAS) and
the measured peak. Prints one JSON line per shape."""
import argparse
import json

import torch

from common import time_ms
from hippolm_b200.ops import cuda_ops as co, nvfp4_cuda, fp4_gemm
from hippolm_b200.utils.timing import load_measured_peaks

SHAPES = [(8192, 8192, 8192), (16384, 4096, 4096), (16384, 28672, 4096), (16384, 4096, 14336), (4096, 14336, 16384)]


def _cublaslt_nvfp4_tflops(M, N, K, xp, xs, wp, ws):
    """Throughput of the library's block-scaled FP4 GEMM (``torch._scaled_mm`` on float4_e2m1fn_x2 operands with e4m3
    scales in the 128x4 tile layout) as a measured FP4 reference; None where this torch build has no such path."""
    try:
        from hippolm_b200.ops import fp4_gemm as fg
        a4 = xp.view(torch.float4_e2m1fn_x2)
        b4 = wp.view(torch.float4_e2m1fn_x2)
        sa = fg.tile_scales(xs, M, K).view(torch.float8_e4m3fn)
        sb = fg.tile_scales(ws, N, K).view(torch.float8_e4m3fn)
        fn = lambda: torch._scaled_mm(a4, b4.t(), sa, sb, out_dtype=torch.bfloat16)
        fn()
        torch.cuda.synchronize()
        ms = time_ms(fn, flush=False)
        return round(2.0 * M * N * K / ms / 1e9, 1)
    except Exception as ex:                                           # noqa: BLE001
        print(json.dumps({"cublaslt_nvfp4": f"unavailable: {type(ex).__name__}: {str(ex)[:160]}"}), flush=True)
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", type=str, default="", help="M,N,K: run only this shape")
    ap.add_argument("--profile", type=str, default="", help="nt|nn|tn|nvfp4|nvfp4_pair: launch only this kernel a few times (for ncu)")
    cli = ap.parse_args()
    shapes = [tuple(int(v) for v in cli.shape.split(","))] if cli.shape else SHAPES
    if cli.profile:
        M, N, K = shapes[0]
        a = torch.randn(M, K, device="cuda").bfloat16(); b = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
        bt, at = b.t().contiguous(), a.t().contiguous()
        if cli.profile in ("nvfp4", "nvfp4_pair"):
            xp, xs, xg = nvfp4_cuda.quantize(a); wp, ws, wg = nvfp4_cuda.quantize(b)
            sfa, sfb = fp4_gemm.tile_scales(xs, M, K), fp4_gemm.tile_scales(ws, N, K)
            mm = fp4_gemm.fp4_matmul_pair if cli.profile == "nvfp4_pair" else fp4_gemm.fp4_matmul_tiled
            fn = lambda: mm(xp, sfa, xg, wp, sfb, wg)
        else:
            fn = {"nt": lambda: co.gemm_nt(a, b), "nn": lambda: co.gemm_nn(a, bt), "tn": lambda: co.gemm_tn(at, bt)}[cli.profile]
        for _ in range(4):
            fn()
        torch.cuda.synchronize()
        return
    pk = load_measured_peaks()
    for (M, N, K) in shapes:
        a = torch.randn(M, K, device="cuda").bfloat16(); b = (0.05 * torch.randn(N, K, device="cuda")).bfloat16()
        bt, at = b.t().contiguous(), a.t().contiguous()
        fl = 2.0 * M * N * K
        rec = {"M": M, "N": N, "K": K}
        for name, fn in (("nt", lambda: co.gemm_nt(a, b)), ("nn", lambda: co.gemm_nn(a, bt)),
                         ("tn", lambda: co.gemm_tn(at, bt)),
                         ("nt_1sm", lambda: co._gemm(a, b, 0, M, N, K, kernel="1sm")),
                         ("nn_1sm", lambda: co._gemm(a, bt, 1, M, N, K, kernel="1sm")),
                         ("tn_1sm", lambda: co._gemm(at, bt, 2, M, N, K, kernel="1sm")),
                         ("cublas", lambda: a @ b.t())):
            ms = time_ms(fn, flush=False)
            rec[name + "_tflops"] = round(fl / ms / 1e9, 1)
        if K % 256 == 0:
            xp, xs, xg = nvfp4_cuda.quantize(a); wp, ws, wg = nvfp4_cuda.quantize(b)
            sfa, sfb = fp4_gemm.tile_scales(xs, M, K), fp4_gemm.tile_scales(ws, N, K)
            ms = time_ms(lambda: fp4_gemm.fp4_matmul_tiled(xp, sfa, xg, wp, sfb, wg), flush=False)
            rec["nvfp4_tflops"] = round(fl / ms / 1e9, 1)
            if M >= 256 and N >= 256:
                try:                                                  # CTA-pair kernel (256x256 tiles)
                    ms = time_ms(lambda: fp4_gemm.fp4_matmul_pair(xp, sfa, xg, wp, sfb, wg), flush=False)
                    rec["nvfp4_pair_tflops"] = round(fl / ms / 1e9, 1)
                except RuntimeError as ex:
                    rec["nvfp4_pair"] = f"failed: {str(ex)[:120]}"
            lib_tf = _cublaslt_nvfp4_tflops(M, N, K, xp, xs, wp, ws)
            if lib_tf is not None:
                # measured library FP4 throughput at the same shape: the denominator for the FP4 kernel's fraction
                rec["cublaslt_nvfp4_tflops"] = lib_tf
                rec["nvfp4_frac_of_cublaslt"] = round(rec["nvfp4_tflops"] / lib_tf, 3)
        rec["bf16_frac_of_" + pk["source"] + "_peak"] = round(rec["nt_tflops"] / pk["bf16_tflops"], 3)
        print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
