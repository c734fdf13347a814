#!/usr/bin/env python
"""python scripts/eval_server.py --config X.yml --checkpoint ckpt.pt [--port 8000] [--max_batch 8]

Also takes the options of the reference's server (``scripts/eval_server.py:495-520``): ``--tokenizer DIR``, ``--model-id``,
``--device``, ``--dtype`` and the size overrides ``--hidden-size --num-layers --num-blocks --num-heads --head-dim
--intermediate-size`` (applied over the configuration file)."""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    import torch
    from hippolm_b200.cli import parse_args
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.data.tokenizer import load_tokenizer
    from hippolm_b200.serve.eval_server import EvalService, build_model_and_load, serve
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True); ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--host", default="127.0.0.1"); ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max_new_tokens", type=int, default=256)
    ap.add_argument("--max_batch", type=int, default=8, help="requests decoded together (those waiting in the queue)")
    ap.add_argument("--tokenizer", default=None, help="tokenizer directory (default: tokenizer_path of the configuration)")
    ap.add_argument("--model-id", dest="model_id", default="hippolm", help="model id reported by /v1/models")
    ap.add_argument("--device", default=None, help="cuda | cpu (default: cuda when there is one)")
    ap.add_argument("--dtype", default=None, choices=["fp32", "fp16", "bf16"], help="default: bf16 on a GPU, fp32 on the CPU")
    sizes = ("hidden_size", "num_layers", "num_blocks", "num_heads", "head_dim", "intermediate_size")
    for k in sizes:
        ap.add_argument("--" + k.replace("_", "-"), dest=k, type=int, default=None)
    a = ap.parse_args(argv)
    args = parse_args(["--config", a.config])
    for k in sizes:
        if getattr(a, k) is not None:
            setattr(args, k, getattr(a, k))
    dev = torch.device(a.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dtype = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16,
             None: torch.bfloat16 if dev.type == "cuda" else torch.float32}[a.dtype]
    model = build_model_and_load(a.checkpoint, HippoConfig.from_namespace(args), dev, dtype)
    svc = EvalService(model, load_tokenizer(a.tokenizer or args.tokenizer_path), model_name=a.model_id,
                      max_new_tokens=a.max_new_tokens, max_batch=a.max_batch)
    srv = serve(svc, a.host, a.port)
    print(f"serving on http://{a.host}:{a.port}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.shutdown()


if __name__ == "__main__":
    main()
