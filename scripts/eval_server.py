#!/usr/bin/env python
"""python scripts/eval_server.py --config X.yml --checkpoint ckpt.pt [--port 8000] [--max_batch 8]"""
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
    a = ap.parse_args(argv)
    args = parse_args(["--config", a.config])
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model = build_model_and_load(a.checkpoint, HippoConfig.from_namespace(args), dev,
                                 torch.bfloat16 if dev.type == "cuda" else torch.float32)
    svc = EvalService(model, load_tokenizer(args.tokenizer_path), max_new_tokens=a.max_new_tokens, max_batch=a.max_batch)
    srv = serve(svc, a.host, a.port)
    print(f"serving on http://{a.host}:{a.port}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.shutdown()


if __name__ == "__main__":
    main()
