"""Model state-dict layout, fused-projection equivalence, checkpoint save/load/prune/resume, NVFP4 module API,
teardown, watchdog, env and GPU selection."""
import json
import os
import time

import pytest
import torch

from hippolm_b200.config import HippoConfig
from hippolm_b200.models.model import HippoModel, shift_targets
from hippolm_b200.models.nvfp4_linear import NVFP4Linear, repack_nvfp4_weights
from hippolm_b200.optim.optimizers import build_param_groups
from hippolm_b200.train import checkpoint as ck


def _cfg(**kw):
    base = dict(vocab_size=128, hidden_size=32, num_heads=2, head_dim=16, num_layers=4, num_blocks=2, intermediate_size=64)
    base.update(kw)
    return HippoConfig(**base)


def test_state_dict_key_layout():
    m = HippoModel(_cfg(use_short_conv=True))
    keys = set(m.state_dict().keys())
    for k in ("embed_tokens.weight", "norm.weight", "lm_head.weight", "attn_res.query", "attn_res.norm.weight",
              "layers.0.attn_norm.weight", "layers.0.attn.qkv_proj.weight", "layers.0.attn.fg_first.weight",
              "layers.0.attn.f_proj1.weight", "layers.0.attn.g_proj1.weight", "layers.0.attn.g_proj1.bias",
              "layers.0.attn.b_proj.weight", "layers.0.attn.A_log", "layers.0.attn.dt_bias",
              "layers.0.attn.o_norm.weight", "layers.0.attn.o_proj.weight", "layers.0.attn.q_conv1d.weight",
              "layers.0.ffn_norm.weight", "layers.0.ffn.gate_up_proj.weight", "layers.0.ffn.down_proj.weight",
              "layers.3.attn.qkv_proj.weight", "layers.3.attn.o_proj.weight"):
        assert k in keys, k
    assert not any("in_proj_weight" in k for k in keys)
    assert HippoModel(_cfg(tie_word_embeddings=True)).state_dict().keys().isdisjoint({"lm_head.weight"})
    nv = HippoModel(_cfg(ffn_nvfp4=True, ffn_nvfp4_no_bf16_master=True)).state_dict()
    assert {"layers.0.ffn.gate_up_proj.packed_weight", "layers.0.ffn.gate_up_proj.scales",
            "layers.0.ffn.gate_up_proj.global_scale"} <= set(nv.keys())


def test_state_dict_roundtrip_restores_fused_projection():
    a, b = HippoModel(_cfg(), seed=1), HippoModel(_cfg(), seed=2)
    b.load_state_dict(a.state_dict())
    assert torch.equal(a.layers[0].attn.in_proj_weight, b.layers[0].attn.in_proj_weight)
    ids = torch.randint(0, 128, (64,))
    assert torch.allclose(a(ids, ids)["loss"], b(ids, ids)["loss"])


def test_fused_projection_equals_split_projections():
    torch.manual_seed(0)
    m = HippoModel(_cfg())
    att = m.layers[0].attn
    sd = m.state_dict()
    x = torch.randn(10, 32)
    fused = x @ att.in_proj_weight.t()
    qkv = x @ sd["layers.0.attn.qkv_proj.weight"].t()
    fg = x @ sd["layers.0.attn.fg_first.weight"].t()
    b = x @ sd["layers.0.attn.b_proj.weight"].t()
    assert torch.allclose(fused[:, :att.n_real], torch.cat([qkv, fg, b], 1), atol=1e-6)
    gu = m.layers[0].ffn.gate_up_proj.weight
    assert gu.shape == (128, 32)


def test_shift_targets_and_varlen_isolation():
    lab = torch.arange(8)
    assert shift_targets(lab).tolist() == [1, 2, 3, 4, 5, 6, 7, -100]
    assert shift_targets(lab, 4).tolist() == [1, 2, 3, -100, 5, 6, 7, -100]
    m = HippoModel(_cfg()).eval()
    ids = torch.randint(0, 128, (96,))
    cu = torch.tensor([0, 40, 96], dtype=torch.int32)
    full = m(ids, cu_seqlens=cu)["logits"]
    second = m(ids[40:], cu_seqlens=torch.tensor([0, 56], dtype=torch.int32))["logits"]
    assert torch.allclose(full[40:], second, atol=1e-4)           # documents do not see each other


def test_generate_and_kda_state_carry():
    m = HippoModel(_cfg(full_attn_interval=0)).eval()
    out = m.generate(torch.tensor([1, 2, 3]), max_new_tokens=4)
    assert out.shape[0] == 7 and out[:3].tolist() == [1, 2, 3]
    ids = torch.randint(0, 128, (64,))
    whole = m(ids)["logits"]
    first = m(ids[:32])
    second = m(ids[32:], kda_states=first["kda_states"])["logits"]
    assert torch.allclose(whole[32:], second, atol=1e-4)          # chunked step with carried state == one pass


def test_nvfp4_linear_chunk_api_and_update():
    torch.manual_seed(0)
    lin = NVFP4Linear(64, 48, no_master=True, act_quant=False)
    assert lin.packed_weight.shape == (48, 32) and lin.scales.shape == (48, 4) and lin.global_scale.shape == (1,)
    assert not list(lin.parameters())
    w0 = lin.material_chunk(0, 48, torch.float32)
    x = torch.randn(5, 64, requires_grad=True)
    y = lin(x)
    assert torch.allclose(y, x @ w0.t(), atol=1e-4)
    y.sum().backward()
    assert lin.grad_w is not None and lin.grad_w.shape == (48, 64) and x.grad is not None
    upd = torch.sign(w0[:16]) * 0.01         # towards zero: the tensor scale stays, untouched rows keep their bytes
    lin.stochastic_rounding = False          # round-to-nearest: the per-element error bound below is deterministic
    lin.decay_and_apply_chunk(0, 16, upd, lr=1.0, wd_factor=1.0)
    w1 = lin.material_chunk(0, 48).float()
    assert (w1[:16] - (w0[:16] - upd)).abs().max() < 0.05 and torch.equal(w1[16:], w0[16:])
    assert list(lin.chunk_ranges(20)) == [(0, 20), (20, 40), (40, 48)]
    lin.commit_bf16_view(torch.randn(48, 64))
    sd = lin.state_dict()
    lin2 = NVFP4Linear(64, 48, no_master=True)
    lin2.load_state_dict(sd)
    assert torch.equal(lin2.material_bf16_view(), lin.material_bf16_view())
    ste = NVFP4Linear(64, 48, no_master=False, dtype=torch.float32)
    ste(torch.randn(3, 64)).sum().backward()
    assert ste.weight.grad is not None
    model = HippoModel(_cfg(ffn_nvfp4=True, ffn_nvfp4_no_bf16_master=True))
    assert repack_nvfp4_weights(model) == 8


def test_checkpoint_roundtrip_prune_and_latest(tmp_path):
    m = HippoModel(_cfg())
    muon, adamw = build_param_groups(m)
    for p in m.parameters():
        p.grad = torch.randn_like(p)
    muon.step(); adamw.step()
    d = str(tmp_path / "checkpoints")
    for step in (1, 5, 12, 30):
        ck.save_checkpoint(m, muon, adamw, step, 1.5, ck.checkpoint_path(d, step))
    payload = torch.load(ck.checkpoint_path(d, 30), weights_only=False)
    assert {"step", "model_state_dict", "optimizer_state_dict", "loss", "scaler_state_dict"} <= set(payload)
    assert set(payload["optimizer_state_dict"]) == {"muon", "adamw"} and payload["model_state_dict"]
    assert ck.find_latest_checkpoint(d).endswith("checkpoint_step_30.pt")
    ck.prune_old_checkpoints(d, 2)
    assert [s for s, _ in ck.list_checkpoints(d)] == [12, 30]
    ck.prune_old_checkpoints(d, 0)
    assert len(ck.list_checkpoints(d)) == 2
    m2 = HippoModel(_cfg(), seed=9)
    mu2, ad2 = build_param_groups(m2)
    step, loss = ck.load_checkpoint(ck.checkpoint_path(d, 30), m2, mu2, ad2)
    assert step == 30 and loss == 1.5
    assert torch.equal(m2.norm.weight, m.norm.weight) and mu2.entries[0].step == 1
    assert not ck.is_sharded_state_dict(payload["model_state_dict"])


def test_training_run_checkpoint_and_resume(tmp_path):
    from hippolm_b200.cli import parse_args
    from hippolm_b200.train.loop import setup_worker, run_training_loop
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = str(tmp_path / "run")
    os.makedirs(run)
    a = parse_args(["--config", os.path.join(root, "configs/test/checkpoint.yml")])
    res = run_training_loop(setup_worker(a, run_dir=run))
    assert res["steps"] == 4 and all(l == l for l in res["losses"])
    assert [s for s, _ in ck.list_checkpoints(os.path.join(run, "checkpoints"))] == [3]
    lines = [json.loads(l) for l in open(os.path.join(run, "metrics.jsonl"))]
    assert len(lines) == 4 and {"loss", "lr_muon", "grad_norm", "tok_per_s", "step_ms"} <= set(lines[0])
    a = parse_args(["--config", os.path.join(root, "configs/test/checkpoint.yml"), "--resume", "latest", "--max_steps", "6",
                    "--mb_timing", "-1"])
    ctx = setup_worker(a, run_dir=run)
    assert ctx.step == 4
    res = run_training_loop(ctx)
    assert res["steps"] == 6
    # --mb_timing: the phase split goes to the metrics and, as a Chrome trace, to logs/trace_rank0.json
    lines = [json.loads(l) for l in open(os.path.join(run, "metrics.jsonl"))]
    assert "phases_ms" in lines[-1] and lines[-1]["phases_ms"]
    tr = json.load(open(os.path.join(run, "logs", "trace_rank0.json")))["traceEvents"]
    ph = [e for e in tr if e["ph"] == "X"]
    assert ph and {e["args"]["step"] for e in ph} == {4, 5} and all(e["dur"] > 0 for e in ph)
    assert set(lines[-1]["phases_ms"]) <= {e["name"] for e in ph}


def test_non_finite_gradients_skip_update_and_clear(tmp_path):
    from hippolm_b200.cli import build_parser
    from hippolm_b200.train.loop import setup_worker, train_step, teardown_worker
    from hippolm_b200.data.loaders import dummy_dataloader
    a = build_parser().parse_args([])
    a.vocab_size, a.hidden_size, a.num_heads, a.head_dim, a.num_layers, a.intermediate_size = 128, 32, 2, 16, 2, 64
    a.full_attn_interval = 0
    loader = dummy_dataloader(1, 64, 128)
    ctx = setup_worker(a, data_iter=loader)
    with torch.no_grad():
        ctx.model.norm.weight[0] = float("nan")
    w0 = ctx.model.layers[0].ffn.down_proj.weight.detach().clone()
    out = train_step(ctx, next(loader))
    assert out["found_inf"] and torch.equal(w0, ctx.model.layers[0].ffn.down_proj.weight)
    assert all(p.grad is None for p in ctx.model.parameters())     # accumulators are cleared on the skip path
    teardown_worker(ctx); teardown_worker(ctx); teardown_worker(None)


def test_watchdog_detects_stall(tmp_path):
    from hippolm_b200.train.watchdog import StepWatchdog
    hits = []
    wd = StepWatchdog(0.1, str(tmp_path), 0, on_stall=lambda s, g: hits.append((s, g)), poll_s=0.02)
    wd.start(); wd.beat(3)
    time.sleep(0.35)
    wd.close()
    assert hits and hits[0][0] == 3 and os.path.exists(tmp_path / "heartbeat.rank0.json")


def test_env_and_gpu_selection(tmp_path, monkeypatch):
    from hippolm_b200 import env
    from hippolm_b200.launch import select_gpus
    p = tmp_path / ".env"
    p.write_text("# c\nFOO_X=1\nNCCL_IB_DISABLE=0\nBAD LINE\nQ='quoted'\n")
    e = {"NCCL_IB_DISABLE": "1"}
    loaded = env.load_dotenv(str(p), e)
    assert loaded == {"FOO_X": "1", "Q": "quoted"} and e["NCCL_IB_DISABLE"] == "1"
    env.pin_nccl_environment(e)
    assert e["NCCL_P2P_LEVEL"] == "NVL"
    assert env.get_cache_dir({"HIPPOLM_CACHE_DIR": "/x"}) == "/x"
    assert env.get_cache_dir({}).endswith(os.path.join(".cache", "hippolm", "datasets"))
    free = [50000, 1000, 50000, 50000, 50000, 50000, 100, 50000]
    assert select_gpus(10240, query=lambda: free) == [2, 3, 4, 5]
    assert select_gpus(10240, want=2, query=lambda: free) == [2, 3]
    assert select_gpus(10240, query=lambda: [0, 0]) == []
    assert select_gpus(10, query=lambda: [100] * 8) == list(range(8))


def test_final_checkpoint_when_the_run_ends_between_periodic_ones(tmp_path):
    from hippolm_b200.cli import parse_args
    from hippolm_b200.train.loop import setup_worker, run_training_loop
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = str(tmp_path / "run")
    os.makedirs(run)
    a = parse_args(["--config", os.path.join(root, "configs/test/checkpoint.yml"), "--max_steps", "3",
                    "--checkpoint_keep_last_n", "5"])
    res = run_training_loop(setup_worker(a, run_dir=run))
    assert res["steps"] == 3
    assert [s for s, _ in ck.list_checkpoints(os.path.join(run, "checkpoints"))] == [1, 2]      # periodic, then final
    a = parse_args(["--config", os.path.join(root, "configs/test/checkpoint.yml"), "--resume", "latest", "--max_steps", "4",
                    "--checkpoint_keep_last_n", "5"])
    ctx = setup_worker(a, run_dir=run)
    assert ctx.step == 3
    run_training_loop(ctx)
    assert [s for s, _ in ck.list_checkpoints(os.path.join(run, "checkpoints"))] == [1, 2, 3]   # step 3 is periodic: once


@pytest.mark.timeout(300)
def test_resume_in_a_later_epoch_of_a_finite_local_dataset(tmp_path):
    """Local jsonl files, several passes over them, a checkpoint in the third pass: the resumed run fast-forwards through
    the finished passes (re-opening the source like the run it continues) and goes on; the end of a pass is sticky
    (a second read after the end-of-data marker returns at once instead of waiting for ever)."""
    import random
    from hippolm_b200.cli import parse_args
    from hippolm_b200.train.loop import setup_worker, run_training_loop
    rng = random.Random(0)
    data = tmp_path / "docs.jsonl"
    with open(data, "w") as f:
        for i in range(8):
            f.write(json.dumps({"content": " ".join(rng.choice(["alpha", "beta", "gamma", "delta", "kernel", "tile"])
                                                     for _ in range(rng.randint(5, 40)))}) + "\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = str(tmp_path / "run")
    os.makedirs(run)
    base = ["--config", os.path.join(root, "configs/test/quick.yml"), "--use_dummy_data", "false", "--synthetic_data", "false",
            "--data_files", str(data), "--tokenizer_path", "builtin", "--vocab_size", "1536", "--batch_size", "2",
            "--seq_len", "128", "--epochs", "50", "--checkpoint_interval", "5", "--checkpoint_keep_last_n", "9"]
    res = run_training_loop(setup_worker(parse_args(base + ["--max_steps", "7"]), run_dir=run))
    assert res["steps"] == 7
    lines = [json.loads(l) for l in open(os.path.join(run, "metrics.jsonl"))]
    assert [l["step"] for l in lines] == list(range(7))
    ctx = setup_worker(parse_args(base + ["--max_steps", "10", "--resume", "latest"]), run_dir=run)
    assert ctx.step == 7 and ctx.extras["epoch"] >= 1               # the final checkpoint of the first run; past pass one
    res = run_training_loop(ctx)
    assert res["steps"] == 10 and all(l == l for l in res["losses"])
    from hippolm_b200.data.prefetch import QueueIterator
    import queue
    q = queue.Queue()
    q.put({"x": 1}); q.put(None)
    it = QueueIterator(q)
    assert next(it) == {"x": 1}
    for _ in range(3):
        with pytest.raises(StopIteration):
            next(it)


def test_resume_latest_finds_the_previous_run(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    import sys
    sys.path.insert(0, os.path.join(root, "scripts"))
    import importlib
    train = importlib.import_module("train")
    out = str(tmp_path / "output")
    cfg = os.path.join(root, "configs/test/checkpoint.yml")
    os.environ.pop("HIPPO_RUN_TS", None)
    os.environ["HIPPO_RUN_TS"] = "20200101_000000"
    run1 = train.main(["--config", cfg, "--output_dir", out, "--max_steps", "4"])
    os.environ["HIPPO_RUN_TS"] = "20200101_000100"
    try:
        run2 = train.main(["--config", cfg, "--output_dir", out, "--max_steps", "6", "--resume", "latest"])
    finally:
        os.environ.pop("HIPPO_RUN_TS", None)
    assert run1 != run2
    steps = [json.loads(l)["step"] for l in open(os.path.join(run2, "metrics.jsonl"))]
    assert steps == [4, 5], steps                                    # continued, not restarted
    assert train.latest_checkpoint_of_previous_runs(str(tmp_path / "nothing")) is None
