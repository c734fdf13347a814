"""Child process of ``test_reference_cli.py``: the reference's own argument parser on its own configuration files (and a
few command lines); the parsed namespaces go to a JSON file."""
import glob
import json
import os
import sys


def command_lines(ref_root):
    cfgs = sorted(glob.glob(os.path.join(ref_root, "configs", "*.yml")) + glob.glob(os.path.join(ref_root, "configs", "test", "*.yml")))
    lines = [["--config", c] for c in cfgs]
    base = os.path.join(ref_root, "configs", "base.yml")
    lines += [["--config", base, "--learning_rate", "0.123", "--muon_lr", "0.5", "--seq_len", "4096"],
              # (a boolean with the value "false" is left out: the reference's ``type=bool`` reads any non-empty string as
              # true; here "false" means false)
              ["--config", os.path.join(ref_root, "configs", "test", "quick.yml"), "--tp_size", "4", "--use_short_conv", "true",
               "--use_dummy_data", "--tp_sim"],
              []]
    return lines


def main():
    ref_root, out = sys.argv[1], sys.argv[2]
    sys.path.insert(0, ref_root)
    from scripts.cli import parse_args
    res = []
    for argv in command_lines(ref_root):
        ns = vars(parse_args(list(argv)))
        res.append({k: v for k, v in ns.items() if isinstance(v, (int, float, str, bool, type(None), dict, list))})
    with open(out, "w") as f:
        json.dump(res, f)


if __name__ == "__main__":
    main()
