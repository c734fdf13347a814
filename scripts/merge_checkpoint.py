#!/usr/bin/env python
"""python scripts/merge_checkpoint.py --config X.yml <checkpoints/checkpoint_step_N.pt> <out.pt>

Puts the per-rank model shards of a tensor-parallel run (the files beside the canonical checkpoint file, listed in its
manifest) back together into one plain checkpoint: what a TP = 1 run writes, what the eval server and ``--init_from`` load.
NVFP4 weights kept without a master copy are written as their exact dequantised values. Optimizer state is not merged."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    from hippolm_b200.cli import parse_args
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.train.reshard import merge_checkpoint
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("checkpoint")
    ap.add_argument("out")
    a = ap.parse_args(argv)
    cfg = HippoConfig.from_namespace(parse_args(["--config", a.config]))
    res = merge_checkpoint(a.checkpoint, cfg, a.out)
    print(f"{a.checkpoint}: step {res['step']}, {len(res['model_state_dict'])} tensors -> {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
