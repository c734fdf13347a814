#!/usr/bin/env python
"""Standalone chunked-KDA forward / forward+backward time.

Shapes of the standalone KDA configuration: B=4, T=8192, H=16, K=V=128, chunk 64, bf16; q,k ~ N(0,1)
L2-normalised per head, v ~ N(0,1), g = -softplus(N(0,1)) per key channel, beta = sigmoid(N(0,1)), fp32
zero initial state, 8 documents of random lengths summing to B*T (cu_seqlens).
Prints one JSON line: {"kda_fwd_ms", "kda_fwd_bwd_ms", ...}."""
import argparse
import json

import torch

from common import time_ms
from hippolm_b200.ops.kda_cuda import _KDAFunction
from hippolm_b200.ops import _ext
from hippolm_b200.ref.kda import l2norm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=4); ap.add_argument("--T", type=int, default=8192)
    ap.add_argument("--H", type=int, default=16); ap.add_argument("--D", type=int, default=128)
    ap.add_argument("--docs", type=int, default=8); ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--profile", action="store_true", help="two forward+backward passes and nothing else (for ncu)")
    a = ap.parse_args()
    torch.manual_seed(0)
    TT = a.B * a.T
    dev = "cuda"
    q = l2norm(torch.randn(TT, a.H, a.D, device=dev)).bfloat16().requires_grad_(True)
    k = l2norm(torch.randn(TT, a.H, a.D, device=dev)).bfloat16().requires_grad_(True)
    v = torch.randn(TT, a.H, a.D, device=dev).bfloat16().requires_grad_(True)
    g = (-torch.nn.functional.softplus(torch.randn(TT, a.H, a.D, device=dev))).requires_grad_(True)
    beta = torch.sigmoid(torch.randn(TT, a.H, device=dev)).requires_grad_(True)
    h0 = torch.zeros(a.docs, a.H, a.D, a.D, device=dev)
    cuts = torch.sort(torch.randperm(TT - 1)[:a.docs - 1] + 1).values
    cu = torch.cat([torch.zeros(1, dtype=torch.long), cuts, torch.tensor([TT])]).to(torch.int32).to(dev)
    do = torch.randn(TT, a.H, a.D, device=dev).bfloat16()

    def fwd():
        with torch.no_grad():
            _KDAFunction.apply(q, k, v, g, beta, h0, cu)

    class Ctx:                                   # stands in for the autograd context: kernels + allocations only
        def save_for_backward(self, *t):
            self.saved_tensors = t

    from hippolm_b200.ops import kda_bwd_cuda
    qd, kd, vd, gd, bd = (t.detach() for t in (q, k, v, g, beta))

    def fwd_bwd():
        ctx = Ctx()
        _KDAFunction.forward(ctx, qd, kd, vd, gd, bd, h0, cu)
        kda_bwd_cuda.backward(ctx, do, None)

    if a.profile:
        fwd_bwd(); fwd_bwd()
        torch.cuda.synchronize()
        return
    f = time_ms(fwd, iters=a.iters)
    fb = time_ms(fwd_bwd, iters=a.iters)
    print(json.dumps({"kda_fwd_ms": round(f, 3), "kda_fwd_bwd_ms": round(fb, 3), "B": a.B, "T": a.T, "H": a.H,
                      "K": a.D, "V": a.D, "docs": a.docs, "dtype": "bf16", "l2": "flushed between iterations",
                      "device_status": list(_ext.device_status())}))


if __name__ == "__main__":
    main()
