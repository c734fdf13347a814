#!/usr/bin/env python
"""Starts the eval server as a subprocess, waits for /health, runs an OpenAI-API evaluation against it
(evalscope when installed, else a completion smoke request) and stops the server (``scripts/eval.py:67-357``).

    python scripts/eval.py --config X.yml --checkpoint ckpt.pt --perplexity --data_files a.txt,b.jsonl [--seq_len 1024]

evaluates offline instead: the perplexity of the checkpoint over local text / jsonl / parquet files, computed by the model's
own loss head in this process (no server, no network)."""
import argparse
import json
import os
import subprocess
import sys
import time
import urllib.request

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def wait_for_health(url: str, timeout_s: float = 120.0) -> bool:
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        try:
            with urllib.request.urlopen(url + "/health", timeout=2) as r:
                if r.status == 200:
                    return True
        except Exception:
            time.sleep(0.5)
    return False


def perplexity_main(a):
    sys.path.insert(0, ROOT)
    import torch
    from hippolm_b200.cli import parse_args
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.data.tokenizer import load_tokenizer
    from hippolm_b200.serve.eval_server import build_model_and_load
    from hippolm_b200.serve.perplexity import evaluate_perplexity, iter_documents
    if not a.data_files:
        raise SystemExit("--perplexity needs --data_files")
    args = parse_args(["--config", a.config])
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    model = build_model_and_load(a.checkpoint, HippoConfig.from_namespace(args), dev,
                                 torch.bfloat16 if dev.type == "cuda" else torch.float32)
    res = evaluate_perplexity(model, load_tokenizer(args.tokenizer_path), iter_documents(a.data_files.split(","), args.text_field),
                              seq_len=a.seq_len, max_tokens=a.max_tokens)
    os.makedirs(a.out, exist_ok=True)
    with open(os.path.join(a.out, "perplexity.json"), "w") as f:
        json.dump(res, f)
    print(json.dumps(res))
    return res


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True); ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--port", type=int, default=8123); ap.add_argument("--datasets", default="mmlu")
    ap.add_argument("--out", default="output/eval")
    ap.add_argument("--perplexity", action="store_true"); ap.add_argument("--data_files", default=None)
    ap.add_argument("--seq_len", type=int, default=1024); ap.add_argument("--max_tokens", type=int, default=None)
    a = ap.parse_args(argv)
    if a.perplexity:
        return perplexity_main(a)
    url = f"http://127.0.0.1:{a.port}"
    cmd = [sys.executable, os.path.join(ROOT, "scripts", "eval_server.py"), "--config", a.config, "--port", str(a.port)]
    if a.checkpoint:
        cmd += ["--checkpoint", a.checkpoint]
    proc = subprocess.Popen(cmd)
    try:
        if not wait_for_health(url):
            raise RuntimeError("eval server did not become healthy")
        os.makedirs(a.out, exist_ok=True)
        try:
            from evalscope import TaskConfig, run_task
            run_task(TaskConfig(model="hippolm-b200", api_url=url + "/v1/chat/completions", eval_type="service",
                                datasets=a.datasets.split(","), work_dir=a.out))
        except ImportError:
            req = urllib.request.Request(url + "/v1/completions", data=json.dumps({"prompt": "Hello", "max_tokens": 8}).encode(),
                                         headers={"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=120) as r:
                res = json.loads(r.read())
            with open(os.path.join(a.out, "smoke.json"), "w") as f:
                json.dump(res, f)
            print("evalscope is not installed; wrote a completion smoke result to", a.out)
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=10)
        except Exception:
            proc.kill()


if __name__ == "__main__":
    main()
