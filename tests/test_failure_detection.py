"""Failure detection without touching a GPU: gloo ranks on CPU, failures made on the host.

* a rank that leaves between steps (exception -> exit notice in the store) is seen by the survivor before its next
  collective;
* a rank that leaves while the survivor is already inside a collective: the short process-group timeout ends the
  collective with an error and the store explains it;
* a rank that goes silent (no heartbeat) is reported after the liveness timeout;
* a checkpoint write error does not stop training.
"""
import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, mode, out_path):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from hippolm_b200.train.liveness import PeerLiveness, PeerLost, default_store
    live = PeerLiveness(default_store(), rank, world, timeout_s=1.5)
    result = {"rank": rank, "steps": 0, "error": None, "reason": None}
    t0 = time.time()
    try:
        for step in range(6):
            live.beat(step)
            if rank == 1 and step == 2:
                if mode == "raise":
                    raise RuntimeError("injected failure on rank 1")
                if mode == "silent":
                    time.sleep(20.0)              # stays alive but stops beating and never joins the collective
                    break
            if mode == "silent" and rank == 0 and step == 2:
                time.sleep(2.0)                   # let the peer's heartbeat age past the liveness timeout
            if mode == "raise" and rank == 0 and step == 2:
                time.sleep(0.5)                   # the peer has left by now: found before the collective
            live.check()
            x = torch.ones(4)
            try:
                dist.all_reduce(x)
            except Exception as ex:               # process-group timeout: ask the store why
                raise live.diagnose(ex)
            result["steps"] = step + 1
    except PeerLost as lost:
        result["error"], result["reason"], result["lost_rank"] = "PeerLost", lost.reason, lost.rank
    except RuntimeError as ex:
        result["error"] = "RuntimeError"
        live.mark_exit(repr(ex))
    finally:
        live.mark_exit("finished")
    result["seconds"] = time.time() - t0
    torch.save(result, out_path + f".{rank}")
    # no destroy_process_group: the peer may be gone, and teardown of a broken gloo group can block


@pytest.mark.parametrize("mode", ["raise", "silent"])
def test_survivor_learns_that_a_peer_left(tmp_path, mode):
    out = str(tmp_path / mode)
    ctx = mp.spawn(_worker, args=(2, _free_port(), mode, out), nprocs=2, join=False)
    deadline = time.time() + 60
    while not os.path.exists(out + ".0") and time.time() < deadline:      # only the survivor's verdict matters
        time.sleep(0.2)
    r0 = torch.load(out + ".0")
    for p in ctx.processes:
        p.join(timeout=2)
        if p.is_alive():
            p.terminate()
    assert r0["error"] == "PeerLost" and r0["lost_rank"] == 1, r0
    assert r0["steps"] == 2 and r0["seconds"] < 30, r0
    if mode == "raise":
        assert "injected failure" in r0["reason"]
    else:
        assert "no heartbeat" in r0["reason"]


def test_diagnose_after_collective_timeout(tmp_path):
    """The peer exits while the survivor is already waiting in the collective."""
    out = str(tmp_path / "late")

    ctx = mp.spawn(_late_worker, args=(2, _free_port(), out), nprocs=2, join=False)
    deadline = time.time() + 60
    while not os.path.exists(out + ".0") and time.time() < deadline:
        time.sleep(0.2)
    r0 = torch.load(out + ".0")
    for p in ctx.processes:
        p.join(timeout=10)
        if p.is_alive():
            p.terminate()
    assert r0["error"] == "PeerLost" and "left during step 1" in r0["reason"], r0
    assert r0["seconds"] < 30


def _late_worker(rank, world, port, out_path):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    from hippolm_b200.train.liveness import PeerLiveness, PeerLost, default_store
    live = PeerLiveness(default_store(), rank, world, timeout_s=30.0)
    t0 = time.time()
    result = {"error": None, "reason": None}
    try:
        for step in range(3):
            live.beat(step)
            live.check()
            if rank == 1 and step == 1:
                time.sleep(0.5)                   # rank 0 is inside the all-reduce by now
                live.mark_exit("left during step 1")
                time.sleep(6.0)                   # keep the store alive (rank 0 hosts it anyway) and never join
                return
            x = torch.ones(2)
            try:
                dist.all_reduce(x)
            except Exception as ex:
                raise live.diagnose(ex)
    except PeerLost as lost:
        result["error"], result["reason"] = "PeerLost", lost.reason
    result["seconds"] = time.time() - t0
    torch.save(result, out_path + f".{rank}")


def test_checkpoint_write_error_does_not_stop_training(tmp_path, monkeypatch):
    from hippolm_b200.cli import build_parser
    from hippolm_b200.train import checkpoint as ckpt
    from hippolm_b200.train.loop import setup_worker, run_training_loop
    from hippolm_b200.data.loaders import synthetic_loader
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        os.environ.pop(k, None)
    a = build_parser().parse_args([])
    a.vocab_size, a.hidden_size, a.num_heads, a.head_dim = 128, 32, 2, 16
    a.num_layers, a.num_blocks, a.intermediate_size = 2, 1, 64
    a.batch_size, a.seq_len, a.max_steps, a.lr_decay_steps = 2, 32, 3, 0
    a.checkpoint_interval = 1
    a.precision = {k: {"dtype": "fp32"} for k in ("model_weights", "gradients", "activations", "muon_momentum",
                                                  "adamw_m", "adamw_v")}

    def boom(*args, **kw):
        raise OSError("disk full (injected)")
    monkeypatch.setattr(ckpt, "save_checkpoint", boom)
    run_dir = str(tmp_path / "run")
    os.makedirs(os.path.join(run_dir, "checkpoints"), exist_ok=True)
    os.makedirs(os.path.join(run_dir, "logs"), exist_ok=True)
    ctx = setup_worker(a, run_dir=run_dir, data_iter=synthetic_loader(2, 32, 128, 0, 8, 32))
    res = run_training_loop(ctx)
    assert res["steps"] == 3 and len(res["losses"]) == 3


def _loop_worker(rank, world, port, out_path):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    torch.set_num_threads(1)
    from hippolm_b200.cli import build_parser
    from hippolm_b200.train.loop import setup_worker, run_training_loop
    from hippolm_b200.train.liveness import PeerLost
    from hippolm_b200.data.loaders import synthetic_loader
    a = build_parser().parse_args([])
    a.vocab_size, a.hidden_size, a.num_heads, a.head_dim = 128, 32, 2, 16
    a.num_layers, a.num_blocks, a.intermediate_size = 2, 1, 64
    a.batch_size, a.seq_len, a.max_steps, a.lr_decay_steps = 4, 32, 6, 0
    a.tp_size, a.dp_size, a.checkpoint_interval = 1, 2, 0
    a.peer_timeout_s, a.dist_timeout_s = 3.0, 5.0
    a.precision = {k: {"dtype": "fp32"} for k in ("model_weights", "gradients", "activations", "muon_momentum",
                                                  "adamw_m", "adamw_v")}

    def data():
        src = synthetic_loader(2, 32, 128, rank, 8, 32)
        for i in range(6):
            if rank == 1 and i == 2:
                raise RuntimeError("injected data failure on rank 1")
            yield next(src)
    t0 = time.time()
    result = {"error": None, "reason": None, "steps": 0}
    ctx = setup_worker(a, run_dir=None, data_iter=data())
    try:
        res = run_training_loop(ctx)
        result["steps"] = res["steps"]
    except PeerLost as lost:
        result.update(error="PeerLost", reason=lost.reason, steps=ctx.step)
    except RuntimeError as ex:
        result.update(error="RuntimeError", reason=str(ex), steps=ctx.step)
    result["seconds"] = time.time() - t0
    torch.save(result, out_path + f".{rank}")


def test_training_loop_reports_lost_peer(tmp_path):
    """Through the public loop: rank 1's data source fails before step 2; rank 0 ends with PeerLost, not a hang."""
    out = str(tmp_path / "loop")
    ctx = mp.spawn(_loop_worker, args=(2, _free_port(), out), nprocs=2, join=False)
    deadline = time.time() + 120
    while not all(os.path.exists(out + f".{r}") for r in range(2)) and time.time() < deadline:
        time.sleep(0.2)
    res = [torch.load(out + f".{r}") for r in range(2)]
    for p in ctx.processes:
        p.join(timeout=10)
        if p.is_alive():
            p.terminate()
    assert res[1]["error"] == "RuntimeError" and "injected data failure" in res[1]["reason"]
    assert res[0]["error"] == "PeerLost" and "injected data failure" in res[0]["reason"], res[0]
    assert res[0]["steps"] == 2 and res[0]["seconds"] < 60


def _flaky_train_worker(args):
    """Worker of the restart test: the first set of workers loses rank 1 at step 3 (an exception on the host, between
    steps); the restarted set runs clean."""
    from hippolm_b200.train import loop
    first_attempt = os.environ.get("HIPPO_RESTART_ATTEMPT") is None
    rank = int(os.environ.get("RANK", "0"))
    if first_attempt and rank == 1:
        real_step = loop.train_step

        def step_that_fails_once(ctx, batch, *rest):
            if ctx.step == 3:
                raise RuntimeError("injected failure on rank 1 at step 3")
            return real_step(ctx, batch, *rest)
        loop.train_step = step_that_fails_once
    ctx = loop.setup_worker(args, run_dir=args.run_dir)
    return loop.run_training_loop(ctx)


def test_launcher_restarts_from_the_latest_checkpoint(tmp_path, monkeypatch):
    """--max_restarts: a worker failure ends the set of workers; the launcher starts a new set that resumes from the newest
    complete checkpoint, and the run reaches its last step."""
    import json
    from hippolm_b200.cli import build_parser
    from hippolm_b200.launch import launch
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "HIPPO_RESTART_ATTEMPT", "HIPPO_TP_SIM"):
        monkeypatch.delenv(k, raising=False)
    a = build_parser().parse_args([])
    a.vocab_size, a.hidden_size, a.num_heads, a.head_dim = 128, 32, 2, 16
    a.num_layers, a.num_blocks, a.intermediate_size = 2, 1, 64
    a.batch_size, a.seq_len, a.max_steps = 2, 64, 6
    a.tp_size, a.dp_size, a.tp_sim = 2, 1, True
    a.use_dummy_data = True
    a.checkpoint_interval, a.checkpoint_keep_last_n = 2, 5
    a.dist_timeout_s = 20.0
    a.max_restarts = 1
    a.precision = {k: {"dtype": "fp32"} for k in ("model_weights", "gradients", "activations", "muon_momentum",
                                                  "adamw_m", "adamw_v")}
    run = tmp_path / "run"
    for sub in ("checkpoints", "logs"):
        os.makedirs(run / sub)
    a.run_dir = str(run)
    launch(_flaky_train_worker, a, 2)
    monkeypatch.delenv("HIPPO_RESTART_ATTEMPT", raising=False)
    monkeypatch.delenv("HIPPO_TP_SIM", raising=False)
    steps = [json.loads(l)["step"] for l in open(run / "metrics.jsonl")]
    # first attempt: steps 0..2 (a checkpoint after step 1); restart: resumes after the checkpoint and finishes
    assert steps[:3] == [0, 1, 2] and steps[-1] == 5, steps
    assert steps[3] == 2, steps
    a.max_restarts = 0
    a.run_dir = str(tmp_path / "run2")
    for sub in ("checkpoints", "logs"):
        os.makedirs(os.path.join(a.run_dir, sub))
    a.resume = None
    with pytest.raises(Exception):
        launch(_flaky_train_worker, a, 2)
