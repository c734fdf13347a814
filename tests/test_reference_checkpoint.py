"""Checkpoint files of the reference (written by its own ``save_checkpoint`` from its own model and optimizers, unmodified
tree, child process) read here: layout detection, the converter script, the eval server's loader and ``--init_from``; and
its pruning rule against the one here on the same directory listings. Needs the copy of the reference tree under
``baseline/_ref`` (skipped without it)."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
WORKER = os.path.join(ROOT, "tests", "reference_checkpoint_worker.py")
needs_ref = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src")), reason="no copy of the reference tree")


def _worker(*argv, cwd):
    r = subprocess.run([sys.executable, WORKER, REF, *argv], capture_output=True, text=True, timeout=900, cwd=cwd)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-3000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


@needs_ref
def test_a_checkpoint_written_by_the_reference_loads_here(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from reference_checkpoint_worker import DIMS
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.serve.eval_server import build_model_and_load
    from hippolm_b200.train.convert import convert_checkpoint_file, detect_layout
    d = tmp_path / "ref_ckpt"
    d.mkdir()
    path = _worker("save", str(d), cwd=str(tmp_path))["path"]
    assert os.path.basename(path) == "checkpoint_step_7.pt"
    ck = torch.load(path, map_location="cpu", weights_only=False)
    assert {"step", "model_state_dict", "optimizer_state_dict", "loss"} <= set(ck) and ck["step"] == 7
    assert detect_layout(ck["model_state_dict"]) == "reference_single"
    exp = torch.load(str(d / "expected.pt"))
    cfg = HippoConfig(full_attn_interval=0, **DIMS)
    # the eval server's loader converts on the fly
    model = build_model_and_load(path, cfg, torch.device("cpu"), torch.float32).eval()
    with torch.no_grad():
        got = model(exp["ids"])["logits"].float()
    assert (got - exp["logits"]).abs().max() < 2e-4 * max(1.0, float(exp["logits"].abs().max()))
    # the converter writes a file that a training run starts from
    out = str(tmp_path / "ours.pt")
    convert_checkpoint_file(path, out)
    conv = torch.load(out, map_location="cpu", weights_only=False)
    assert detect_layout(conv["model_state_dict"]) == "native" and conv["step"] == 7
    from hippolm_b200.models.model import HippoModel
    m2 = HippoModel(cfg)
    m2.load_state_dict(conv["model_state_dict"], strict=True)
    for (n, a), (_, b) in zip(model.state_dict().items(), m2.state_dict().items()):
        assert torch.equal(a.float(), b.float()), n


@needs_ref
def test_pruning_rule_matches_the_reference(tmp_path):
    from hippolm_b200.train.checkpoint import prune_old_checkpoints
    names = ["checkpoint_step_%d.pt" % s for s in (5, 10, 100, 20, 9)] + ["best.pt", "checkpoint_step_x.pt", "notes.txt"]
    keeps = [-1, 0, 1, 3, 10]
    for tag in ("ref", "here"):
        for keep in keeps:
            d = tmp_path / tag / str(keep)
            d.mkdir(parents=True)
            for n in names:
                (d / n).write_bytes(b"0")
    removed_ref = _worker("prune", str(tmp_path / "ref"), cwd=str(tmp_path))["removed"]
    for keep in keeps:
        here = tmp_path / "here" / str(keep)
        removed_here = prune_old_checkpoints(str(here), keep)
        if keep == 0:
            # the reference's function removes every checkpoint at 0, the one just written included (its command-line help
            # promises "keep only the just-saved file"); here 0 keeps all
            assert removed_ref["0"] == 5 and removed_here == 0 and len(os.listdir(here)) == len(names)
            continue
        assert sorted(os.listdir(tmp_path / "ref" / str(keep))) == sorted(os.listdir(here)), keep
        assert removed_ref[str(keep)] == removed_here, keep
