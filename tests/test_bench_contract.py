"""bench.py contract pieces that need no GPU: without a CUDA device the reference arm still answers with one JSON line
and exit code 0 and imports nothing of this package, and the Muon ownership split across data-parallel replicas is
balanced and deterministic."""
import json
import os
import subprocess
import sys

import torch
import torch.nn as nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_answers_without_a_gpu():
    import pytest
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "src")):
        pytest.skip("the reference tree has not been copied to baseline/_ref")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--model", "tiny", "--gpus", "1", "--steps", "1",
                        "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference"
    if not torch.cuda.is_available():
        # the tree imports, but its worker needs a CUDA device: the arm says so instead of failing
        assert "CUDA" in rec["unavailable"]
    else:
        assert rec.get("value", 0) > 0 or rec.get("unavailable")


def test_reference_arm_source_does_not_import_the_package():
    src = open(os.path.join(ROOT, "baseline", "reference_arm.py")).read()
    assert "import hippolm_b200" not in src and "from hippolm_b200" not in src


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
