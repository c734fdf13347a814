"""Benchmark driver around the eval server (the reference's ``scripts/eval.py:67-357``): server life cycle (spawn and wait
for ``/health``, or use a server that already runs), the evalscope task when that package is installed, and a built-in
multiple-choice scorer over local files otherwise (or on request), so that a checkpoint can be scored on a machine without
network or extra packages.

Three ways to reach a server, as in the reference: ``--api-url URL`` (used as given, nothing is started), ``--no-server``
(``http://host:port``, nothing is started), default (start ``scripts/eval_server.py``, wait, stop it afterwards).

Built-in scorer: ``--dataset`` names a ``.jsonl`` file whose rows hold ``question``, ``choices`` (list of strings) and
``answer`` (index or letter), optionally ``subject``. Every row becomes one chat completion ("Answer with the letter only")
with ``--fewshot`` solved rows of the same subject in front; the first stand-alone letter of the reply that names a choice is the prediction. Requests
run ``--batch-size`` at a time so that the server decodes them together."""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import json
import logging
import os
import re
import subprocess
import sys
import time
import urllib.request
from typing import Dict, List, Optional

log = logging.getLogger("hippo.eval")
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
_SIZES = ("hidden_size", "num_layers", "num_blocks", "num_heads", "head_dim", "intermediate_size")
_LETTERS = "ABCDEFGHIJKLMNOPQRSTUVWXYZ"


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="score a checkpoint through the eval server",
                                formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    # model serving (handed to scripts/eval_server.py)
    p.add_argument("--config", required=True); p.add_argument("--checkpoint", default=None)
    p.add_argument("--tokenizer", default=None); p.add_argument("--model-id", dest="model_id", default="hippolm")
    p.add_argument("--dtype", default=None, choices=["fp32", "fp16", "bf16"]); p.add_argument("--device", default=None)
    for k in _SIZES:
        p.add_argument("--" + k.replace("_", "-"), dest=k, type=int, default=None)
    p.add_argument("--max_batch", type=int, default=8, help="requests the server decodes together")
    # server life cycle
    p.add_argument("--host", default="127.0.0.1"); p.add_argument("--port", type=int, default=18080)
    p.add_argument("--no-server", dest="no_server", action="store_true", help="use http://host:port, start nothing")
    p.add_argument("--api-url", dest="api_url", default=None, help="chat-completions URL of a running server")
    p.add_argument("--server-log", dest="server_log", default=None, help="default: <work-dir>/eval_server.log")
    # benchmark
    p.add_argument("--dataset", "--datasets", dest="dataset", default="mmlu",
                   help="an evalscope benchmark id, or a .jsonl file for the built-in multiple-choice scorer")
    p.add_argument("--subset", default=None, help="comma-separated subsets (subjects)")
    p.add_argument("--fewshot", type=int, default=None); p.add_argument("--limit", type=int, default=None)
    p.add_argument("--batch-size", dest="batch_size", type=int, default=8)
    p.add_argument("--max-tokens", dest="max_new", type=int, default=64)
    p.add_argument("--dataset-dir", dest="dataset_dir", default=os.path.expanduser("~/.cache/modelscope/hub/datasets"))
    p.add_argument("--dataset-hub", dest="dataset_hub", default="modelscope", choices=["modelscope", "huggingface"])
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--work-dir", "--out", dest="work_dir", default="output/eval")
    p.add_argument("--ignore-errors", dest="ignore_errors", action="store_true")
    p.add_argument("--debug", action="store_true")
    # offline perplexity (no server)
    p.add_argument("--perplexity", action="store_true"); p.add_argument("--data_files", default=None)
    p.add_argument("--seq_len", type=int, default=1024); p.add_argument("--max_tokens", type=int, default=None)
    return p


# ---------------------------------------------------------------------------------------------------- server life cycle
def server_command(a) -> List[str]:
    cmd = [sys.executable, os.path.join(ROOT, "scripts", "eval_server.py"), "--config", a.config, "--host", a.host,
           "--port", str(a.port), "--model-id", a.model_id, "--max_batch", str(a.max_batch),
           "--max_new_tokens", str(max(a.max_new, 1))]
    for flag, val in (("--checkpoint", a.checkpoint), ("--tokenizer", a.tokenizer), ("--dtype", a.dtype), ("--device", a.device)):
        if val:
            cmd += [flag, str(val)]
    for k in _SIZES:
        if getattr(a, k) is not None:
            cmd += ["--" + k.replace("_", "-"), str(getattr(a, k))]
    return cmd


def wait_for_health(url: str, timeout_s: float = 300.0, proc: Optional[subprocess.Popen] = None) -> bool:
    t0 = time.time()
    while time.time() - t0 < timeout_s:
        if proc is not None and proc.poll() is not None:
            return False                                   # the server ended before it answered
        try:
            with urllib.request.urlopen(url, timeout=2) as r:
                if r.status == 200:
                    return True
        except Exception:                                  # noqa: BLE001
            time.sleep(0.5)
    return False


def stop_server(proc: subprocess.Popen, log_file=None) -> None:
    if proc.poll() is None:
        proc.terminate()
        try:
            proc.wait(timeout=15)
        except subprocess.TimeoutExpired:
            proc.kill()
            proc.wait(timeout=15)
    if log_file is not None:
        log_file.close()


# ---------------------------------------------------------------------------------------------------- evalscope
def evalscope_task_kwargs(a, api_url: str) -> Dict:
    """Keyword arguments of ``evalscope.config.TaskConfig`` for these options (greedy, non-streaming chat completions)."""
    ds_args = {}
    if a.subset:
        ds_args["subset_list"] = [s.strip() for s in a.subset.split(",") if s.strip()]
    if a.fewshot is not None and a.fewshot >= 0:
        ds_args["few_shot_num"] = int(a.fewshot)
    return dict(model=a.model_id, model_id=a.model_id, api_url=api_url, api_key="EMPTY", eval_type="service",
                datasets=[a.dataset], dataset_args={a.dataset: ds_args} if ds_args else {}, dataset_dir=a.dataset_dir,
                dataset_hub=a.dataset_hub, limit=a.limit, eval_batch_size=a.batch_size,
                generation_config={"max_tokens": a.max_new, "temperature": 0.0, "stream": False}, work_dir=a.work_dir,
                seed=a.seed, ignore_errors=a.ignore_errors, debug=a.debug)


def run_evalscope(a, api_url: str) -> int:
    from evalscope import run_task
    from evalscope.config import TaskConfig
    try:
        res = run_task(TaskConfig(**evalscope_task_kwargs(a, api_url)))
    except SystemExit as e:                                # evalscope leaves through sys.exit on configuration errors
        log.error("evalscope exited with code %s", e.code)
        return e.code if isinstance(e.code, int) else 1
    for r in (res if isinstance(res, list) else [res]):
        if isinstance(r, dict):
            log.info("benchmark %s: %s", r.get("benchmark_name", "?"), r.get("metrics", r))
    return 0


# ---------------------------------------------------------------------------------------------------- built-in scorer
def load_choice_rows(path: str, subsets: Optional[List[str]] = None) -> List[Dict]:
    rows = []
    with open(path) as f:
        for ln, line in enumerate(f, 1):
            line = line.strip()
            if not line:
                continue
            r = json.loads(line)
            ans = r["answer"]
            if isinstance(ans, str):
                ans = _LETTERS.index(ans.strip().upper()[0]) if not ans.strip().isdigit() else int(ans)
            if not (0 <= int(ans) < len(r["choices"])):
                raise ValueError(f"{path}:{ln}: answer {r['answer']!r} is not one of the {len(r['choices'])} choices")
            row = {"question": str(r["question"]), "choices": [str(c) for c in r["choices"]], "answer": int(ans),
                   "subject": str(r.get("subject", "all"))}
            if not subsets or row["subject"] in subsets:
                rows.append(row)
    return rows


def _format_row(r: Dict, with_answer: bool) -> str:
    body = r["question"].strip() + "\n" + "\n".join(f"{_LETTERS[i]}. {c}" for i, c in enumerate(r["choices"])) + "\nAnswer:"
    return body + (f" {_LETTERS[r['answer']]}\n\n" if with_answer else "")


def choice_prompt(row: Dict, shots: List[Dict]) -> str:
    head = "The following are multiple choice questions. Answer with the letter only.\n\n"
    return head + "".join(_format_row(s, True) for s in shots) + _format_row(row, False)


def parse_choice(text: str, n_choices: int) -> Optional[int]:
    """First letter of the reply that stands alone ("B", "B.", "(b)", "answer: C") and names one of the choices."""
    for m in re.finditer(r"(?<![A-Za-z])([A-Za-z])(?![A-Za-z])", text or ""):
        i = _LETTERS.find(m.group(1).upper())
        if 0 <= i < n_choices:
            return i
    return None


def _chat(api_url: str, model_id: str, prompt: str, max_new: int, timeout: float = 600.0) -> str:
    body = {"model": model_id, "messages": [{"role": "user", "content": prompt}], "max_tokens": max_new, "temperature": 0.0,
            "stream": False}
    req = urllib.request.Request(api_url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())["choices"][0]["message"]["content"]


def run_choice_file(a, api_url: str, ask=None) -> Dict:
    """Scores the rows of ``a.dataset`` (a .jsonl file) through chat completions; ``ask(prompt) -> reply`` replaces the
    HTTP call (tests). Writes ``<work-dir>/report.json`` and ``predictions.jsonl``; returns the report."""
    subsets = [s.strip() for s in a.subset.split(",") if s.strip()] if a.subset else None
    rows = load_choice_rows(a.dataset, subsets)
    by_subject: Dict[str, List[Dict]] = {}
    for r in rows:
        by_subject.setdefault(r["subject"], []).append(r)
    k = max(0, a.fewshot or 0)
    work = []
    for subj, rs in sorted(by_subject.items()):
        shots, test = rs[:k], rs[k:]                        # the first rows of a subject are its solved examples
        if a.limit is not None:
            test = test[:a.limit]
        work += [(subj, r, shots) for r in test]
    ask = ask or (lambda prompt: _chat(api_url, a.model_id, prompt, a.max_new))
    replies: List[Optional[str]] = [None] * len(work)

    def one(i):
        try:
            replies[i] = ask(choice_prompt(work[i][1], work[i][2]))
        except Exception as e:                             # noqa: BLE001
            if not a.ignore_errors:
                raise
            log.warning("request %d failed: %r", i, e)

    with cf.ThreadPoolExecutor(max_workers=max(1, a.batch_size)) as pool:
        list(pool.map(one, range(len(work))))
    per: Dict[str, List[int]] = {}
    os.makedirs(a.work_dir, exist_ok=True)
    with open(os.path.join(a.work_dir, "predictions.jsonl"), "w") as f:
        for (subj, r, _), reply in zip(work, replies):
            pred = parse_choice(reply, len(r["choices"])) if reply is not None else None
            per.setdefault(subj, []).append(int(pred == r["answer"]))
            f.write(json.dumps({"subject": subj, "question": r["question"], "answer": r["answer"], "prediction": pred,
                                "reply": reply}) + "\n")
    n = sum(len(v) for v in per.values())
    report = {"dataset": a.dataset, "model": a.model_id, "fewshot": k, "n": n,
              "accuracy": (sum(sum(v) for v in per.values()) / n) if n else None,
              "chance": (sum(1.0 / len(r["choices"]) for _, r, _ in work) / n) if n else None,
              "subjects": {s: {"n": len(v), "accuracy": sum(v) / len(v)} for s, v in sorted(per.items())},
              "seed": a.seed}
    with open(os.path.join(a.work_dir, "report.json"), "w") as f:
        json.dump(report, f, indent=1)
    log.info("accuracy %.4f over %d questions (chance %.4f)", report["accuracy"] or 0.0, n, report["chance"] or 0.0)
    return report


# ---------------------------------------------------------------------------------------------------- offline perplexity
def run_perplexity(a) -> Dict:
    import torch
    from ..cli import parse_args
    from ..config import HippoConfig
    from ..data.tokenizer import load_tokenizer
    from .eval_server import build_model_and_load
    from .perplexity import evaluate_perplexity, iter_documents
    if not a.data_files:
        raise SystemExit("--perplexity needs --data_files")
    args = parse_args(["--config", a.config])
    for k in _SIZES:
        if getattr(a, k) is not None:
            setattr(args, k, getattr(a, k))
    dev = torch.device(a.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dtype = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16,
             None: torch.bfloat16 if dev.type == "cuda" else torch.float32}[a.dtype]
    model = build_model_and_load(a.checkpoint, HippoConfig.from_namespace(args), dev, dtype)
    res = evaluate_perplexity(model, load_tokenizer(a.tokenizer or args.tokenizer_path),
                              iter_documents(a.data_files.split(","), args.text_field), seq_len=a.seq_len,
                              max_tokens=a.max_tokens)
    os.makedirs(a.work_dir, exist_ok=True)
    with open(os.path.join(a.work_dir, "perplexity.json"), "w") as f:
        json.dump(res, f)
    print(json.dumps(res))
    return res


# ---------------------------------------------------------------------------------------------------- entry point
def main(argv=None) -> int:
    logging.basicConfig(level=logging.INFO, format="%(asctime)s [%(levelname)s] %(message)s")
    a = build_parser().parse_args(argv)
    if a.perplexity:
        run_perplexity(a)
        return 0
    os.makedirs(a.work_dir, exist_ok=True)
    base = f"http://{a.host}:{a.port}"
    proc = log_file = None
    if a.api_url:
        api_url = a.api_url
    elif a.no_server:
        api_url = base + "/v1/chat/completions"
    else:
        api_url = base + "/v1/chat/completions"
        log_file = open(a.server_log or os.path.join(a.work_dir, "eval_server.log"), "w")
        proc = subprocess.Popen(server_command(a), stdout=log_file, stderr=subprocess.STDOUT)
        if not wait_for_health(base + "/health", proc=proc):
            stop_server(proc, log_file)
            log.error("the eval server did not come up; see %s", log_file.name)
            return 2
    try:
        if os.path.isfile(a.dataset):
            run_choice_file(a, api_url)
            return 0
        try:
            import evalscope  # noqa: F401
        except ImportError:
            # neither a local file nor evalscope: one completion shows that the served model answers
            reply = _chat(api_url, a.model_id, "Hello", min(a.max_new, 8))
            with open(os.path.join(a.work_dir, "smoke.json"), "w") as f:
                json.dump({"reply": reply}, f)
            log.warning("evalscope is not installed and --dataset is not a local .jsonl file; wrote one completion to %s",
                        a.work_dir)
            return 0
        return run_evalscope(a, api_url)
    except Exception:                                      # noqa: BLE001
        log.exception("evaluation failed")
        return 1
    finally:
        if proc is not None:
            stop_server(proc, log_file)
