#!/usr/bin/env python
"""Starts the eval server as a subprocess, waits for /health, runs an OpenAI-API evaluation against it
(evalscope when installed, else a built-in perplexity-free smoke prompt set) and stops the server
(``scripts/eval.py:67-357``)."""
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


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True); ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--port", type=int, default=8123); ap.add_argument("--datasets", default="mmlu")
    ap.add_argument("--out", default="output/eval")
    a = ap.parse_args(argv)
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
