"""bench.py contract pieces that need no GPU: the reference arm answers with one JSON line and exit code 0, and the
Muon ownership split across data-parallel replicas is balanced and deterministic."""
import json
import os
import subprocess
import sys

import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "1",
                        "--warmup", "1"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and rec["unavailable"]


def test_muon_dp_owner_assignment_is_balanced():
    from hippolm_b200.optim.optimizers import Muon
    opt = Muon(lr=0.02, momentum_dtype=torch.float32, dp_shard=True)
    shapes = [(64, 256), (64, 64), (256, 64), (64, 64), (64, 64), (128, 64), (64, 256), (8, 64)]
    for i, sh in enumerate(shapes):
        opt.add_param(nn.Parameter(torch.zeros(*sh)), f"w{i}")
    owners = opt._dp_owners(2)
    assert owners == opt._dp_owners(2) and set(owners) == {0, 1}
    load = [sum(a * b for (a, b), o in zip(shapes, owners) if o == r) for r in range(2)]
    assert abs(load[0] - load[1]) <= max(a * b for a, b in shapes)
