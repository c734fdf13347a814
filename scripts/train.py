#!/usr/bin/env python
"""Training entry point: ``python scripts/train.py --config configs/X.yml [--flag ...]``.

Single process -> inline worker; ``--nproc N`` (or tp_size*dp_size > 1) -> one spawned process per
GPU; under ``torchrun`` each rank runs this file directly.
"""
import datetime
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from hippolm_b200.cli import parse_args                      # noqa: E402
from hippolm_b200.env import configure_runtime_environment   # noqa: E402


def create_output_dir(base: str) -> str:
    ts = os.environ.get("HIPPO_RUN_TS") or datetime.datetime.now().strftime("%Y%m%d_%H%M%S")
    os.environ["HIPPO_RUN_TS"] = ts
    run = os.path.join(base, ts)
    for sub in ("checkpoints", "logs", "eval"):
        os.makedirs(os.path.join(run, sub), exist_ok=True)
    return run


def _worker(args):
    from hippolm_b200.train.loop import setup_worker, run_training_loop
    ctx = setup_worker(args, run_dir=args.run_dir)
    return run_training_loop(ctx)


def latest_checkpoint_of_previous_runs(base: str, exclude: str = None):
    """Newest complete checkpoint among the run directories under ``base`` (newest run first), or None."""
    from hippolm_b200.train.checkpoint import find_latest_checkpoint
    if not os.path.isdir(base):
        return None
    for run in sorted((d for d in os.listdir(base) if os.path.isdir(os.path.join(base, d, "checkpoints"))), reverse=True):
        if exclude and os.path.abspath(os.path.join(base, run)) == os.path.abspath(exclude):
            continue
        p = find_latest_checkpoint(os.path.join(base, run, "checkpoints"))
        if p:
            return p
    return None


def train(args):
    from hippolm_b200.launch import launch
    args.run_dir = create_output_dir(args.output_dir)
    if getattr(args, "resume", None) in ("latest", "auto"):
        # every invocation gets a run directory of its own: "latest" means the newest checkpoint of the earlier runs under
        # the same output directory (inside a run, a restarted set of workers finds its own checkpoints first)
        prev = latest_checkpoint_of_previous_runs(args.output_dir, exclude=args.run_dir)
        if prev:
            print(f"resuming from {prev}", flush=True)
            args.resume = prev
    world = args.nproc or max(1, args.tp_size * max(1, args.dp_size))
    launch(_worker, args, world)
    return args.run_dir


def main(argv=None):
    args = parse_args(argv)
    configure_runtime_environment(args.cache_dir)
    return train(args)


if __name__ == "__main__":
    main()
