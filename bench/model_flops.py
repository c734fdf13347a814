#!/usr/bin/env python
"""Analytic FLOP count of one training step of a hybrid KDA / attention decoder, and the model-FLOP utilisation a
measured throughput corresponds to (no GPU needed).

    python bench/model_flops.py --tokens_per_s 14796 --gpus 1

Counts matmul FLOPs as 2 per multiply-add: 6 x parameters per token for the linears (forward + dX + dW), causal attention
4 S d H / 2 per token forward and 3.5x that with backward, the chunked KDA products, the LCE head and the Newton-Schulz
iterations of Muon (5 iterations; Gram products counted at half cost when the symmetric kernel applies).
Peaks come from MEASURED_PEAKS.json when present (cuBLAS bf16 burst and sustained), else the stated fallback."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from hippolm_b200.utils.flops import step_flops             # noqa: E402
from hippolm_b200.utils.timing import load_measured_peaks   # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=4096); ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--head_dim", type=int, default=128); ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--attn_interval", type=int, default=4); ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=128256); ap.add_argument("--seq_len", type=int, default=8192)
    ap.add_argument("--seqs_per_gpu", type=int, default=16); ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--tokens_per_s", type=float, default=0.0)
    a = ap.parse_args()
    tokens = a.seqs_per_gpu * a.gpus * a.seq_len
    per_tok, total_tok, muon = step_flops(a.hidden, a.heads, a.head_dim, a.layers, a.attn_interval, a.ffn, a.vocab,
                                          a.seq_len, tokens)
    pk = load_measured_peaks()
    rec = {"tokens_per_step": tokens, "gflop_per_token": {k: round(v / 1e9, 3) for k, v in per_tok.items()},
           "model_pflop_per_step": round(total_tok / 1e15, 3), "muon_pflop_per_step": round(muon / 1e15, 3),
           "peak_source": pk["source"], "bf16_tflops_burst": pk["bf16_tflops"]}
    if a.tokens_per_s > 0:
        step_s = tokens / a.tokens_per_s
        model_rate = total_tok / step_s / 1e12 / a.gpus
        all_rate = (total_tok + muon) / step_s / 1e12 / a.gpus
        rec.update({"s_per_step": round(step_s, 3), "model_tflops_per_gpu": round(model_rate, 1),
                    "model_plus_muon_tflops_per_gpu": round(all_rate, 1),
                    "mfu_of_" + pk["source"] + "_burst_peak": round(model_rate / pk["bf16_tflops"], 3)})
        sus = pk.get("bf16_tflops_sustained")
        if sus:
            rec["mfu_of_" + pk["source"] + "_sustained_peak"] = round(model_rate / sus, 3)
    print(json.dumps(rec))


if __name__ == "__main__":
    main()
