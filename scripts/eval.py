#!/usr/bin/env python
"""Scores a checkpoint: starts the eval server (or uses a running one), runs an evalscope benchmark or the built-in
multiple-choice scorer over a local .jsonl file against it, stops the server (the reference's ``scripts/eval.py:67-357``,
same option names).

    python scripts/eval.py --config X.yml --checkpoint ckpt.pt --dataset mmlu --limit 100
    python scripts/eval.py --config X.yml --checkpoint ckpt.pt --dataset questions.jsonl --fewshot 5
    python scripts/eval.py --config X.yml --checkpoint ckpt.pt --perplexity --data_files a.txt,b.jsonl [--seq_len 1024]

The last form evaluates offline: the perplexity of the checkpoint over local text / jsonl / parquet files, computed by the
model's own loss head in this process (no server, no network)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    from hippolm_b200.serve.eval_driver import main as run
    return run(argv)


if __name__ == "__main__":
    sys.exit(main())
