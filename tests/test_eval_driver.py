"""Benchmark driver (``hippolm_b200/serve/eval_driver.py``, ``scripts/eval.py``): option surface of the reference's driver,
the evalscope task arguments, the built-in multiple-choice scorer (scoring logic with a scripted model, and end to end: the
script starts a server for a tiny random model, scores a local file through chat completions and stops the server)."""
import json
import os
import socket
import subprocess
import sys

from hippolm_b200.serve import eval_driver as ed

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rows(path, n=12):
    with open(path, "w") as f:
        for i in range(n):
            f.write(json.dumps({"question": f"What is {i} + 1?", "choices": [str(i), str(i + 1), str(i + 2), str(i + 3)],
                                "answer": "B" if i % 2 else 1, "subject": "even" if i % 2 == 0 else "odd"}) + "\n")


def test_option_surface_and_evalscope_arguments():
    a = ed.build_parser().parse_args(
        ["--config", "c.yml", "--checkpoint", "k.pt", "--tokenizer", "tok", "--model-id", "m", "--dtype", "bf16", "--device",
         "cpu", "--hidden-size", "64", "--num-layers", "2", "--num-blocks", "1", "--num-heads", "2", "--head-dim", "32",
         "--intermediate-size", "128", "--host", "127.0.0.1", "--port", "18081", "--server-log", "s.log", "--dataset", "mmlu",
         "--subset", "anatomy, virology", "--fewshot", "0", "--limit", "4", "--batch-size", "2", "--max-tokens", "16",
         "--dataset-dir", "/d", "--dataset-hub", "huggingface", "--seed", "7", "--work-dir", "w", "--ignore-errors", "--debug"])
    kw = ed.evalscope_task_kwargs(a, "http://x/v1/chat/completions")
    assert kw["datasets"] == ["mmlu"] and kw["dataset_args"] == {"mmlu": {"subset_list": ["anatomy", "virology"], "few_shot_num": 0}}
    assert kw["generation_config"] == {"max_tokens": 16, "temperature": 0.0, "stream": False}
    assert (kw["limit"], kw["eval_batch_size"], kw["seed"], kw["ignore_errors"], kw["debug"]) == (4, 2, 7, True, True)
    assert kw["model"] == kw["model_id"] == "m" and kw["api_key"] == "EMPTY" and kw["dataset_hub"] == "huggingface"
    cmd = ed.server_command(a)
    for flag, val in (("--checkpoint", "k.pt"), ("--tokenizer", "tok"), ("--model-id", "m"), ("--dtype", "bf16"),
                      ("--device", "cpu"), ("--hidden-size", "64"), ("--head-dim", "32"), ("--port", "18081")):
        assert cmd[cmd.index(flag) + 1] == val
    b = ed.build_parser().parse_args(["--config", "c.yml", "--datasets", "gsm8k", "--out", "o"])      # earlier spellings
    assert b.dataset == "gsm8k" and b.work_dir == "o" and ed.evalscope_task_kwargs(b, "u")["dataset_args"] == {}


def test_builtin_scorer_counts_right_and_wrong_answers(tmp_path):
    data = str(tmp_path / "q.jsonl")
    _rows(data)
    a = ed.build_parser().parse_args(["--config", "c.yml", "--dataset", data, "--fewshot", "2", "--work-dir", str(tmp_path / "w"),
                                      "--batch-size", "3"])
    prompts = []

    def ask(prompt):                       # answers "B" on even subjects only
        prompts.append(prompt)
        last = prompt.rsplit("What is ", 1)[1]
        return " B." if int(last.split(" ")[0]) % 2 == 0 else "I think (d)"

    rep = ed.run_choice_file(a, "unused", ask=ask)
    assert rep["n"] == 8 and rep["fewshot"] == 2                            # 2 of the 6 rows per subject are the examples
    assert rep["subjects"]["even"] == {"n": 4, "accuracy": 1.0} and rep["subjects"]["odd"] == {"n": 4, "accuracy": 0.0}
    assert rep["accuracy"] == 0.5 and rep["chance"] == 0.25
    assert all(p.count("Answer:") == 3 and p.rstrip().endswith("Answer:") for p in prompts)
    # solved examples come from the same subject and are not scored
    even = [p for p in prompts if "What is 4 + 1?" in p.rsplit("Answer:", 2)[1]]
    assert even and "What is 0 + 1?" in even[0] and "What is 2 + 1?" in even[0] and "What is 1 + 1?" not in even[0]
    preds = [json.loads(l) for l in open(tmp_path / "w" / "predictions.jsonl")]
    assert len(preds) == 8 and {p["prediction"] for p in preds} == {1, 3}
    assert json.load(open(tmp_path / "w" / "report.json"))["accuracy"] == 0.5
    assert ed.parse_choice("", 4) is None and ed.parse_choice("z", 4) is None and ed.parse_choice("(c)", 4) == 2
    # subsets, limits
    a2 = ed.build_parser().parse_args(["--config", "c.yml", "--dataset", data, "--subset", "odd", "--limit", "3",
                                       "--work-dir", str(tmp_path / "w2")])
    rep2 = ed.run_choice_file(a2, "unused", ask=lambda p: "B")
    assert rep2["n"] == 3 and list(rep2["subjects"]) == ["odd"] and rep2["accuracy"] == 1.0


def test_script_scores_a_local_file_through_its_own_server(tmp_path):
    data = str(tmp_path / "q.jsonl")
    _rows(data, 6)
    cfg = tmp_path / "m.yml"
    cfg.write_text("vocab_size: 1536\nhidden_size: 32\nnum_heads: 2\nhead_dim: 16\nnum_layers: 2\nnum_blocks: 1\n"
                   "intermediate_size: 64\ntokenizer_path: builtin\n")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    work = tmp_path / "w"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "scripts", "eval.py"), "--config", str(cfg), "--port", str(port),
                        "--device", "cpu", "--dtype", "fp32", "--dataset", data, "--max-tokens", "2", "--batch-size", "3",
                        "--work-dir", str(work)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    rep = json.load(open(work / "report.json"))
    assert rep["n"] == 6 and 0.0 <= rep["accuracy"] <= 1.0 and rep["chance"] == 0.25
    assert os.path.getsize(work / "eval_server.log") > 0
    # the server is gone: nothing listens on its port
    with socket.socket() as s:
        assert s.connect_ex(("127.0.0.1", port)) != 0
