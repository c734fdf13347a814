#!/usr/bin/env python
"""python scripts/convert_checkpoint.py <reference checkpoint .pt> <output .pt>

Rewrites the model weights of a checkpoint of the reference (its single-GPU layout or its one-device tensor-parallel
layout) into this framework's plain ``layers.N.*`` layout; the result loads with ``model.load_state_dict`` and the eval
server (which also converts on the fly) into a model built with ``full_attn_interval: 0`` and the same dimensions. Optimizer
state is not carried over."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        print(__doc__)
        return 2
    from hippolm_b200.train.convert import convert_checkpoint_file
    info = convert_checkpoint_file(argv[0], argv[1])
    print(f"{argv[0]}: layout {info['layout']}, step {info['step']}, {info['tensors']} tensors -> {argv[1]}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
