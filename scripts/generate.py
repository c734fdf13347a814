#!/usr/bin/env python
"""python scripts/generate.py --config X.yml [--checkpoint ckpt.pt] --prompt "text" [--max_new_tokens 64]
                              [--temperature 0.8 --top_k 40 --top_p 0.95]

Completes a prompt with a checkpoint (this framework's, a tensor-parallel run's canonical file, or the reference's) in this
process: incremental decoding on the GPU when one is visible, else on the CPU."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    import torch
    from hippolm_b200.cli import parse_args
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.data.tokenizer import load_tokenizer
    from hippolm_b200.serve.eval_server import build_model_and_load
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True); ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--prompt", required=True); ap.add_argument("--max_new_tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0); ap.add_argument("--top_k", type=int, default=0)
    ap.add_argument("--top_p", type=float, default=1.0); ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    args = parse_args(["--config", a.config])
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model = build_model_and_load(a.checkpoint, HippoConfig.from_namespace(args), dev,
                                 torch.bfloat16 if dev.type == "cuda" else torch.float32)
    tok = load_tokenizer(args.tokenizer_path)
    torch.manual_seed(a.seed)
    ids = tok.encode(a.prompt, add_special_tokens=False) or [getattr(tok, "eos_token_id", 0) or 0]
    out = model.generate(torch.tensor(ids, dtype=torch.long, device=dev), a.max_new_tokens, temperature=a.temperature,
                         top_k=a.top_k, top_p=a.top_p, eos_token_id=getattr(tok, "eos_token_id", None))
    text = tok.decode(out[len(ids):].tolist(), skip_special_tokens=True)
    print(text)
    return text


if __name__ == "__main__":
    main()
