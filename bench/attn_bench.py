#!/usr/bin/env python
"""Causal varlen flash attention forward / forward+backward time and achieved TFLOPS."""
import json

import torch

from common import time_ms
from hippolm_b200 import ops


def main():
    for (B, S, H, D) in [(2, 8192, 32, 128), (4, 4096, 16, 128)]:
        T = B * S
        q, k, v = (torch.randn(T, H, D, device="cuda").bfloat16().requires_grad_(True) for _ in range(3))
        do = torch.randn(T, H, D, device="cuda").bfloat16()
        cu = torch.arange(0, T + 1, S, dtype=torch.int32, device="cuda")

        def fwd():
            with torch.no_grad():
                ops.causal_attention(q, k, v, cu)

        def fb():
            ops.causal_attention(q, k, v, cu).backward(do)
        f, t = time_ms(fwd), time_ms(fb)
        fl = 4.0 * B * S * S * D * H / 2
        print(json.dumps({"B": B, "S": S, "H": H, "D": D, "fwd_ms": round(f, 3), "fwd_bwd_ms": round(t, 3),
                          "fwd_tflops": round(fl / f / 1e9, 1), "fwd_bwd_tflops": round(3.5 * fl / t / 1e9, 1)}))


if __name__ == "__main__":
    main()
