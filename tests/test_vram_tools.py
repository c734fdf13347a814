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


def test_phase_memory_tracks_the_peak_inside_every_phase():
    """PhaseTimer + PhaseMemory with scripted allocator counters: the peak counter is reset at the start of a phase, read at
    its end, and the maximum of the whole run survives the resets."""
    from hippolm_b200.utils.timing import PhaseTimer
    from hippolm_b200.utils.vram import PhaseMemory
    state = {"alloc": 0, "peak": 0, "resets": 0}

    def alloc(n):
        state["alloc"] += n
        state["peak"] = max(state["peak"], state["alloc"])

    def reset():
        state["peak"] = state["alloc"]; state["resets"] += 1

    mem = PhaseMemory(readers={"allocated": lambda: state["alloc"], "reserved": lambda: 2 * state["alloc"],
                               "peak": lambda: state["peak"], "reset_peak": reset, "driver_used": lambda: state["alloc"] + 5})
    mib = 2 ** 20
    alloc(10 * mib)                                     # weights, before any phase
    for step in range(2):
        t = PhaseTimer(enabled=True, step=step, memory=mem)
        with t.phase("fwd_bwd"):
            alloc(100 * mib * (step + 1)); alloc(-90 * mib * (step + 1))
        with t.phase("muon"):
            alloc(30 * mib); alloc(-30 * mib)
        with t.phase("fwd_bwd"):                        # a phase may occur twice in a step (micro-batches)
            alloc(20 * mib); alloc(-20 * mib)
    assert state["resets"] == 6 and len(mem.rows) == 6
    assert mem.step_summary(0) == {"fwd_bwd": 110.0, "muon": 50.0}
    assert mem.step_summary(1)["fwd_bwd"] == 220.0
    tab = {r["phase"]: r for r in mem.table()}
    assert list(tab) == ["fwd_bwd", "muon"] and tab["fwd_bwd"]["step"] == 1 and tab["fwd_bwd"]["peak_mib"] == 220.0
    assert tab["fwd_bwd"]["allocated_mib"] == 40.0 and tab["fwd_bwd"]["reserved_mib"] == 80.0
    assert mem.run_peak == 220 * mib
    # without a GPU the default readers give zeros and nothing fails
    z = PhaseMemory(torch.device("cpu")); z.begin(); assert z.record("x")["peak"] == 0


def test_snapshot_classification_by_component():
    from hippolm_b200.utils.vram import classify_block, classify_snapshot
    pk = "/site/hippolm_b200/"

    def blk(size, *frames, state="active_allocated"):
        return {"size": size, "state": state, "frames": [{"filename": f, "name": n, "line": 1} for f, n in frames]}

    snap = {"segments": [{"blocks": [
        blk(1000, ("/torch/nn/modules/linear.py", "__init__"), (pk + "models/model.py", "__init__")),
        blk(400, (pk + "ops/kda_cuda.py", "forward"), (pk + "models/model.py", "forward")),
        blk(300, (pk + "ops/cuda_ops.py", "rmsnorm"), (pk + "models/model.py", "forward")),
        blk(250, (pk + "optim/optimizers.py", "add_param")),
        blk(200, (pk + "models/model.py", "_VocabParallelLCE.forward")),
        blk(150, (pk + "parallel/symm.py", "alloc")),
        blk(120, ("/torch/utils/checkpoint.py", "forward"), (pk + "models/model.py", "forward")),
        blk(100, (pk + "ops/attn_cuda.py", "forward")),
        blk(50, ("/somewhere/else.py", "f")),
        blk(7, ),
        blk(9999, (pk + "ops/kda_cuda.py", "forward"), state="inactive"),
    ]}]}
    rows = classify_snapshot(snap)
    got = {r["class"]: r["bytes"] for r in rows}
    assert got == {"model.weight": 1000, "kda.saved": 400, "norm.saved": 300, "optimizer.state": 250, "lce_head": 200,
                   "comm.workspace": 150, "checkpoint.input": 120, "attention.saved": 100, "other": 50, "<no stack>": 7}
    assert [r["bytes"] for r in rows] == sorted((r["bytes"] for r in rows), reverse=True)
    assert rows[0]["largest"].startswith(pk + "models/model.py") and classify_block([]) == "<no stack>"


def test_profile_command_runs_steps_and_reports_phases(tmp_path, capsys):
    import json
    import os
    from hippolm_b200.utils.vram import _main
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = str(tmp_path / "prof")
    assert _main(["profile", "--config", os.path.join(root, "configs", "test", "quick.yml"), "--steps", "2", "--out", out]) == 0
    res = json.load(open(os.path.join(out, "vram_profile.json")))
    assert {r["phase"] for r in res["phases"]} >= {"h2d", "fwd_bwd", "gradnorm", "muon", "adamw", "zero"} and res["steps"] == 2
    lines = [json.loads(l) for l in open(os.path.join(out, "metrics.jsonl"))] if os.path.exists(os.path.join(out, "metrics.jsonl")) \
        else [json.loads(l) for l in open(os.path.join(out, "logs", "metrics.jsonl"))]
    assert all("phases_peak_mb" in l and "fwd_bwd" in l["phases_peak_mb"] for l in lines)


def test_training_metrics_carry_model_flops_and_utilisation(tmp_path):
    """Every logged step has the analytic model TFLOP/s per GPU and its fraction of the GEMM peak; the numbers follow
    from the FLOP model and the logged step time."""
    import json
    import os
    import sys
    from hippolm_b200.cli import parse_args
    from hippolm_b200.config import HippoConfig
    from hippolm_b200.utils.flops import config_step_flops, step_flops
    from hippolm_b200.utils.timing import load_measured_peaks
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "scripts"))
    import train as train_script
    args = parse_args(["--config", os.path.join(root, "configs", "test", "quick.yml"), "--max_steps", "2",
                       "--output_dir", str(tmp_path)])
    run = train_script.train(args)
    lines = [json.loads(l) for l in open(os.path.join(run, "metrics.jsonl"))]
    cfg = HippoConfig.from_namespace(args)
    pk = load_measured_peaks()
    for l in lines:
        _, total, _ = config_step_flops(cfg, args.seq_len, l["tokens"])
        want = total / l["step_ms"] * 1e3 / 1e12
        assert abs(l["model_tflops_per_gpu"] - want) <= 0.006 + 1e-3 * want
        assert abs(l["mfu"] - want / pk["bf16_tflops_sustained"]) < 1e-3
    # the 7B benchmark model: ~52.5 GFLOP per token, dominated by the linears
    per_tok, total, muon = step_flops(4096, 32, 128, 32, 4, 14336, 128256, 8192, 131072)
    assert 50e9 < sum(per_tok.values()) < 55e9 and per_tok["linears"] > 0.85 * sum(per_tok.values()) and muon < 0.1 * total
