"""Data parallelism together with gradient offload and with fully masked windows (CPU, gloo, spawned ranks).

* dp=2 with ``offload_grads`` (overlap hooks requested and not requested): the gradients uploaded from the host
  accumulators must be reduced over the replicas, so the replicas end with identical weights that match a single
  process run on the concatenated batch.
* one replica's last micro-batch window fully masked: every replica must still issue the same collectives (no hang, no
  mismatched buckets) and match the single-process run.
* the per-step check of the device status word: a bounded wait that ran out raises and clears the gradients.
"""
import os
import types

import pytest
import torch
import torch.multiprocessing as mp

from test_parallel_parity import _args, _batch, _free_port


def _masked_batch(dp_rank, dp, mask_rank):
    b = _batch(dp_rank, dp)
    if dp_rank == mask_rank or (dp == 1 and mask_rank is not None):
        labels = b["labels"].clone()
        n = labels.numel()
        if dp == 1:
            # the single-process oracle sees the concatenated batch: mask what the masked replica would mask
            half = n // 2
            s = mask_rank * half
            labels[s + half - 64:s + half] = -100
        else:
            labels[n - 64:] = -100
        b = dict(b, labels=labels)
    return b


def _run(rank, world, port, dp, out_path, offload, overlap, mask_rank, mbs):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    torch.set_num_threads(1)
    from hippolm_b200.train.loop import setup_worker, train_step, teardown_worker
    a = _args(1, dp, to_owner=(dp > 1))          # the default: Muon gradients are reduced to their owning replica only
    a.offload_grads, a.dp_overlap, a.dist_timeout_s = offload, overlap, 60
    a.micro_batch_size = mbs
    ctx = setup_worker(a, run_dir=None, data_iter=iter(()))
    losses, gnorms = [], []
    for _ in range(2):
        out = train_step(ctx, _masked_batch(ctx.mesh.dp_rank, dp, mask_rank)); ctx.step += 1
        losses.append(float(out["loss"])); gnorms.append(float(out["grad_norm"]))
    sd = {k: v.detach().clone() for k, v in ctx.model.state_dict().items()}
    torch.save({"losses": losses, "gnorms": gnorms, "sd": sd}, out_path + f".{rank}")
    teardown_worker(ctx)


def _launch(tmp_path, dp, offload=False, overlap=True, mask_rank=None, mbs=0, tag=""):
    out = str(tmp_path / f"o_dp{dp}_{int(offload)}{int(overlap)}{mask_rank}{mbs}{tag}")
    if dp == 1:
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            os.environ.pop(k, None)
        _run(0, 1, _free_port(), 1, out, offload, overlap, mask_rank, mbs)
    else:
        mp.spawn(_run, args=(dp, _free_port(), dp, out, offload, overlap, mask_rank, mbs), nprocs=dp, join=True)
    return [torch.load(out + f".{r}", weights_only=False) for r in range(dp)]


@pytest.mark.parametrize("overlap", [True, False])
def test_dp2_with_gradient_offload_reduces_the_uploaded_gradients(tmp_path, overlap):
    ref = _launch(tmp_path, 1)[0]
    res = _launch(tmp_path, 2, offload=True, overlap=overlap)
    for r in res:
        for a, b in zip(r["losses"], ref["losses"]):
            assert abs(a - b) < 2e-3, (r["losses"], ref["losses"])       # bf16 host accumulators
        assert abs(r["gnorms"][0] - ref["gnorms"][0]) < 1e-2 * max(1.0, ref["gnorms"][0])
    for k in res[0]["sd"]:
        assert torch.equal(res[0]["sd"][k], res[1]["sd"][k]), f"replicas diverged on {k}"
    for k in ("norm.weight", "layers.0.ffn.down_proj.weight", "embed_tokens.weight"):
        # bf16 host accumulators perturb near-zero gradients, which Adam's normalisation turns into +-lr: compare on average
        assert (res[0]["sd"][k] - ref["sd"][k]).abs().mean() < 5e-4, k


def test_dp2_last_window_fully_masked_on_one_replica(tmp_path):
    # two windows per replica (128 tokens, windows of 64); replica 1's last window has no valid target
    ref = _launch(tmp_path, 1, mask_rank=1, mbs=64)[0]
    res = _launch(tmp_path, 2, mask_rank=1, mbs=64)
    for r in res:
        for a, b in zip(r["losses"], ref["losses"]):
            assert abs(a - b) < 2e-4, (r["losses"], ref["losses"])
    for k in res[0]["sd"]:
        assert torch.equal(res[0]["sd"][k], res[1]["sd"][k]), f"replicas diverged on {k}"


def test_fused_status_word_is_checked_every_step(monkeypatch):
    import logging
    from hippolm_b200.train import loop
    from hippolm_b200.ops import _ext
    cleared, zeroed = [], []
    monkeypatch.setattr(_ext, "device_status", lambda: (3, 7, 11, 1))
    monkeypatch.setattr(_ext, "clear_device_status", lambda: cleared.append(1))
    opt = types.SimpleNamespace(zero_grad=lambda: zeroed.append(1))
    ctx = types.SimpleNamespace(step=5, muon=opt, adamw=opt, logger=logging.getLogger("t"), extras={"fused_comm": True})
    with pytest.raises(loop.FusedCommTimeout) as ei:
        loop._check_fused_status(ctx)
    assert "code=3" in str(ei.value) and cleared == [1] and len(zeroed) == 2
    monkeypatch.setattr(_ext, "device_status", lambda: (0, 0, 0, 0))
    loop._check_fused_status(ctx)            # clean status: no exception


def test_fused_trial_with_an_expired_wait_falls_back(monkeypatch):
    """The first-use timing of a fused op doubles as a probe: when the device status word says that a bounded wait ran out
    during the trial, the status is cleared, the workspace counters are reset and the trial counts as failed."""
    import types
    import torch
    from hippolm_b200.parallel import fused
    from hippolm_b200.ops import _ext
    calls = {"cleared": 0, "reset": 0}
    status = {"v": (5, 101, 3, 1)}
    monkeypatch.setattr(_ext, "device_status", lambda: status["v"])
    monkeypatch.setattr(_ext, "clear_device_status", lambda: (calls.__setitem__("cleared", calls["cleared"] + 1),
                                                              status.__setitem__("v", (0, 0, 0, 0)))[0])
    ws = types.SimpleNamespace(mesh=types.SimpleNamespace(device=torch.device("cpu")),
                               reset_counters=lambda: calls.__setitem__("reset", calls["reset"] + 1))
    assert fused._trial_failed(ws, None) is True
    assert calls == {"cleared": 1, "reset": 1}
    assert fused._trial_failed(ws, None) is False          # clean status: nothing to do
    assert calls == {"cleared": 1, "reset": 1}


def _dp_finite_worker(rank, world, port, data, run_dir):
    import os
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port), "HIPPO_TP_SIM": "1"})
    import torch
    torch.set_num_threads(1)
    from hippolm_b200.cli import build_parser
    from hippolm_b200.train.loop import setup_worker, run_training_loop
    a = build_parser().parse_args([])
    a.vocab_size, a.hidden_size, a.num_heads, a.head_dim = 1536, 32, 2, 16
    a.num_layers, a.num_blocks, a.intermediate_size = 2, 1, 64
    a.batch_size, a.seq_len, a.max_steps, a.epochs = 4, 128, 40, 2
    a.tp_size, a.dp_size, a.tp_sim = 1, 2, True
    a.use_dummy_data = a.synthetic_data = False
    a.data_files, a.tokenizer_path, a.dist_timeout_s = data, "builtin", 30.0
    a.precision = {k: {"dtype": "fp32"} for k in ("model_weights", "gradients", "activations", "muon_momentum", "adamw_m", "adamw_v")}
    res = run_training_loop(setup_worker(a, run_dir=run_dir))
    torch.save({"steps": res["steps"], "losses": res["losses"]}, os.path.join(run_dir, f"res.{rank}.pt"))


def test_dp_replicas_end_a_finite_data_pass_together(tmp_path):
    """One local file, two replicas reading every second row; the rows of one replica are much longer, so it has more
    batches per pass. Both end each pass at the same step (agreed by a collective) and the run finishes."""
    import json
    import socket
    import torch
    import torch.multiprocessing as mp
    data = tmp_path / "docs.jsonl"
    with open(data, "w") as f:
        for i in range(40):
            f.write(json.dumps({"content": ("long row " * 40) if i % 2 == 0 else "short"}) + "\n")
    run = tmp_path / "run"
    (run / "logs").mkdir(parents=True)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    mp.spawn(_dp_finite_worker, args=(2, port, str(data), str(run)), nprocs=2, join=True)
    r0, r1 = torch.load(run / "res.0.pt"), torch.load(run / "res.1.pt")
    assert r0["steps"] == r1["steps"] and 0 < r0["steps"] < 40
    assert all(l == l for l in r0["losses"])
