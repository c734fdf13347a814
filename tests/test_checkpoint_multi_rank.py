"""Multi-rank checkpoints (CPU, gloo, tp=2): save, resume and compare; incomplete steps are never picked; a missing shard
or a manifest of another layout is refused instead of silently loading rank 0's weights."""
import json
import os

import pytest
import torch
import torch.multiprocessing as mp

from test_parallel_parity import _args, _batch, _free_port


def _run(rank, world, port, run_dir, mode, out_path):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    torch.set_num_threads(1)
    from hippolm_b200.train.loop import setup_worker, train_step, teardown_worker
    from hippolm_b200.train import checkpoint as ck
    a = _args(2, 1)
    d = os.path.join(run_dir, "checkpoints")
    result = {}
    if mode == "save":
        ctx = setup_worker(a, run_dir=run_dir, data_iter=iter(()))
        for _ in range(2):
            out = train_step(ctx, _batch(0, 1)); ctx.step += 1
        ck.save_checkpoint(ctx.model, ctx.muon, ctx.adamw, 1, float(out["loss"]), ck.checkpoint_path(d, 1),
                           rank=rank, world_size=world, mesh=ctx.mesh)
        out = train_step(ctx, _batch(0, 1)); ctx.step += 1
        result = {"loss3": float(out["loss"]), "sd": {k: v.clone() for k, v in ctx.model.state_dict().items()}}
    elif mode == "resume":
        a.resume = "latest"
        ctx = setup_worker(a, run_dir=run_dir, data_iter=iter(()))
        assert ctx.step == 2
        out = train_step(ctx, _batch(0, 1)); ctx.step += 1
        result = {"loss3": float(out["loss"]), "sd": {k: v.clone() for k, v in ctx.model.state_dict().items()}}
    elif mode == "resume_missing":
        a.resume = ck.checkpoint_path(d, 1)
        try:
            setup_worker(a, run_dir=run_dir, data_iter=iter(()))
            result = {"error": None}
        except FileNotFoundError as ex:
            result = {"error": str(ex)}
        ctx = None
    torch.save(result, out_path + f".{rank}")
    if ctx is not None:
        teardown_worker(ctx)
    else:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


def _launch(tmp_path, mode):
    out = str(tmp_path / f"res_{mode}")
    mp.spawn(_run, args=(2, _free_port(), str(tmp_path / "run"), mode, out), nprocs=2, join=True)
    return [torch.load(out + f".{r}", weights_only=False) for r in range(2)]


def test_tp2_save_resume_and_refusals(tmp_path):
    from hippolm_b200.train import checkpoint as ck
    os.makedirs(tmp_path / "run")
    saved = _launch(tmp_path, "save")
    d = str(tmp_path / "run" / "checkpoints")
    p = ck.checkpoint_path(d, 1)
    man = ck.read_manifest(p)
    assert man["world_size"] == 2 and man["tp"] == 2 and len(man["shards"]) == 2 and ck.is_complete(p)
    resumed = _launch(tmp_path, "resume")
    for r in range(2):
        assert abs(saved[r]["loss3"] - resumed[r]["loss3"]) < 1e-6
        for k in saved[r]["sd"]:
            assert torch.equal(saved[r]["sd"][k], resumed[r]["sd"][k]), (r, k)
    # the shards differ between the ranks (so loading rank 0's file on rank 1 would be a silent error)
    assert not torch.equal(saved[0]["sd"]["layers.0.ffn.down_proj.weight"], saved[1]["sd"]["layers.0.ffn.down_proj.weight"])

    # a later step whose manifest never appeared (interrupted save) is not "latest"
    import shutil
    shutil.copy(p, ck.checkpoint_path(d, 7))
    shutil.copy(p[:-3] + ".rank0.pt", ck.checkpoint_path(d, 7)[:-3] + ".rank0.pt")
    assert not ck.is_complete(ck.checkpoint_path(d, 7))
    assert ck.find_latest_checkpoint(d) == p

    # another layout in the manifest is refused
    class _Mesh:
        tp, dp = 1, 2
    with pytest.raises(ValueError):
        ck.load_checkpoint(p, None, rank=0, world_size=2, mesh=_Mesh())

    # rank 1's shard is gone: rank 1 refuses, and the step no longer counts as complete
    os.remove(p[:-3] + ".rank1.pt")
    assert not ck.is_complete(p)
    res = _launch(tmp_path, "resume_missing")
    assert res[1]["error"] and "rank 1" in res[1]["error"]
