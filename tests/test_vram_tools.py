"""VRAM tooling that needs no GPU: snapshot analysis on a synthetic allocator snapshot, saved-tensor attribution."""
import pickle

import torch
import torch.nn as nn


def test_analyze_snapshot_groups_live_blocks(tmp_path):
    from hippolm_b200.utils.vram import analyze_snapshot
    fr_a = [{"filename": "/x/torch/nn/functional.py", "line": 1, "name": "linear"},
            {"filename": "/x/hippolm_b200/models/model.py", "line": 300, "name": "forward"}]
    fr_b = [{"filename": "/x/hippolm_b200/ops/cuda_ops.py", "line": 25, "name": "_gemm"}]
    snap = {"segments": [{"blocks": [{"size": 100, "state": "active_allocated", "frames": fr_a},
                                     {"size": 50, "state": "inactive", "frames": fr_a},
                                     {"size": 300, "state": "active_allocated", "frames": fr_b}]},
                         {"blocks": [{"size": 25, "state": "active_allocated", "frames": fr_a},
                                     {"size": 7, "state": "active_allocated", "frames": []}]}]}
    p = tmp_path / "snap.pickle"
    p.write_bytes(pickle.dumps(snap))
    for src in (snap, str(p)):
        rows = analyze_snapshot(src)
        assert rows[0]["bytes"] == 300 and "_gemm" in rows[0]["where"]
        assert rows[1]["bytes"] == 125 and rows[1]["blocks"] == 2 and "model.py:300" in rows[1]["where"]
        assert rows[2] == {"where": "<no stack>", "bytes": 7, "blocks": 1}


def test_saved_bytes_by_module_attributes_activations():
    from hippolm_b200.utils.vram import saved_bytes_by_module
    model = nn.Sequential(nn.Linear(16, 64), nn.ReLU(), nn.Linear(64, 8))
    x = torch.randn(4, 16, requires_grad=True)
    rows = saved_bytes_by_module(model, lambda: model(x).sum())
    by = {r["module"]: r["bytes"] for r in rows}
    assert by.get("0", 0) >= 4 * 16 * 4            # the first linear keeps its input
    assert by.get("2", 0) >= 4 * 64 * 4            # the last linear keeps the hidden activations
    assert sum(by.values()) > 0


def test_vram_cli_probe_and_analyze(tmp_path, capsys):
    import os
    import pickle
    from hippolm_b200.utils import vram
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    assert vram._main(["probe", "--config", os.path.join(root, "configs/test/quick.yml"), "--tokens", "128", "--depth", "1"]) == 0
    out = capsys.readouterr().out
    assert "layers" in out and '"saved_mib"' in out
    snap = {"segments": [{"blocks": [{"state": "active_allocated", "size": 4096,
                                      "frames": [{"filename": "/x/hippolm_b200/models/model.py", "line": 7, "name": "forward"}]},
                                     {"state": "inactive", "size": 1 << 20, "frames": []}]}]}
    p = tmp_path / "snap.pickle"
    with open(p, "wb") as f:
        pickle.dump(snap, f)
    assert vram._main(["analyze", str(p), "--top", "3"]) == 0
    assert "model.py:7 forward" in capsys.readouterr().out
