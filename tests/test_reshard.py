"""Tensor-parallel shards <-> plain layout: merging the shards of every TP size gives the TP = 1 model bit for bit (the
initialisation is defined on the full matrices and then sharded), splitting gives the shards back, NVFP4 weights travel as
their exact dequantised values, and a merged multi-rank checkpoint loads into the single-process model / the eval server."""
import os

import pytest
import torch

from hippolm_b200.config import HippoConfig
from hippolm_b200.models.model import HippoModel
from hippolm_b200.parallel import mesh as mesh_mod
from hippolm_b200.train.reshard import merge_tp_state_dicts, split_plain_state_dict

DIMS = dict(vocab_size=256, hidden_size=64, num_heads=4, head_dim=16, num_layers=4, num_blocks=2, intermediate_size=128,
            full_attn_interval=2, use_short_conv=True)


def _model(tp, rank, **kw):
    """The model of one TP rank, built in this process (construction needs the mesh coordinates only, no collective)."""
    mesh_mod._MESH = mesh_mod.Mesh(world_size=tp, rank=rank, tp=tp, dp=1, tp_rank=rank, dp_rank=0)
    try:
        return HippoModel(HippoConfig(**{**DIMS, **kw}), seed=11)
    finally:
        mesh_mod.reset_mesh()


@pytest.mark.parametrize("tp", [2, 4])
@pytest.mark.parametrize("kw", [dict(), dict(tie_word_embeddings=True, use_short_conv=False, safe_gate=True)])
def test_merge_and_split_round_trip(tp, kw):
    cfg = HippoConfig(**{**DIMS, **kw})
    plain = _model(1, 0, **kw).state_dict()
    shards = [_model(tp, r, **kw).state_dict() for r in range(tp)]
    merged = merge_tp_state_dicts(shards, cfg)
    assert set(merged) == set(plain)
    for k in plain:
        assert merged[k].shape == plain[k].shape and torch.equal(merged[k], plain[k]), k
    for r in range(tp):
        back = split_plain_state_dict(plain, cfg, tp, r)
        assert set(back) == set(shards[r])
        for k in back:
            assert torch.equal(back[k], shards[r][k]), (r, k)
        _model(tp, r, **kw).load_state_dict(back, strict=True)
    # and across TP sizes: 4 -> plain -> 2
    if tp == 4:
        two = [_model(2, r, **kw).state_dict() for r in range(2)]
        for r in range(2):
            again = split_plain_state_dict(merged, cfg, 2, r)
            assert all(torch.equal(again[k], two[r][k]) for k in again)


def test_nvfp4_no_master_weights_merge_as_their_values_and_load_back():
    from hippolm_b200 import ops
    kw = dict(ffn_nvfp4=True, ffn_nvfp4_no_bf16_master=True)
    cfg = HippoConfig(**{**DIMS, **kw})
    shards = [_model(2, r, **kw).state_dict() for r in range(2)]
    merged = merge_tp_state_dicts(shards, cfg)
    assert not any(k.endswith("packed_weight") for k in merged)
    k = "layers.1.ffn.down_proj."
    halves = [ops.nvfp4_dequantize(s[k + "packed_weight"], s[k + "scales"], s[k + "global_scale"], torch.bfloat16) for s in shards]
    assert torch.equal(merged[k + "weight"], torch.cat(halves, 1))
    # a no-master model quantises the plain values on load; a bf16-FFN model takes them as they are
    m1 = _model(1, 0, **kw)
    m1.load_state_dict(merged, strict=True)
    got = ops.nvfp4_dequantize(m1.layers[1].ffn.down_proj.packed_weight, m1.layers[1].ffn.down_proj.scales,
                               m1.layers[1].ffn.down_proj.global_scale, torch.float32)
    want = merged[k + "weight"].float()
    assert (got - want).abs().max() <= 0.26 * want.abs().max()          # one more FP4 rounding (new tensor scale), no more
    assert torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0) > 0.99
    _model(1, 0).load_state_dict(merged, strict=True)
    # split with re-quantisation per rank: values that are FP4-representable under the rank's own scale come back exactly
    back = split_plain_state_dict(merged, cfg, 2, 1)
    deq = ops.nvfp4_dequantize(back[k + "packed_weight"], back[k + "scales"], back[k + "global_scale"], torch.bfloat16)
    assert torch.equal(deq, halves[1])
    _model(2, 1, **kw).load_state_dict(back, strict=True)


def _tp_train_worker(rank, world, port, run_dir, init_from):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port), "HIPPO_TP_SIM": "1"})
    torch.set_num_threads(1)
    from hippolm_b200.cli import build_parser
    from hippolm_b200.train.loop import setup_worker, run_training_loop
    a = build_parser().parse_args([])
    for k, v in DIMS.items():
        setattr(a, k, v)
    a.batch_size, a.seq_len, a.max_steps, a.tp_size, a.dp_size, a.tp_sim = 2, 64, 2, world, 1, True
    a.use_dummy_data, a.checkpoint_interval, a.seed = True, 2, 5
    a.precision = {k: {"dtype": "fp32"} for k in ("model_weights", "gradients", "activations", "muon_momentum", "adamw_m", "adamw_v")}
    a.init_from = init_from
    ctx = setup_worker(a, run_dir=run_dir)
    if init_from:
        torch.save({k: v.detach().clone() for k, v in ctx.model.state_dict().items()}, os.path.join(run_dir, f"init_sd.{rank}.pt"))
        from hippolm_b200.train.loop import teardown_worker
        teardown_worker(ctx)
        return
    run_training_loop(ctx)


def test_multi_rank_checkpoint_merges_and_seeds_runs_of_other_sizes(tmp_path):
    """Two gloo ranks train and checkpoint; the merged file loads into the single-process model and the eval server's
    loader, and --init_from starts a one-rank and a two-rank run from it with exactly those weights."""
    import socket
    import torch.multiprocessing as mp
    from hippolm_b200.serve.eval_server import build_model_and_load
    from hippolm_b200.train import checkpoint as ck
    from hippolm_b200.train.reshard import merge_checkpoint

    def port():
        s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p

    run = tmp_path / "run"
    os.makedirs(run / "checkpoints"); os.makedirs(run / "logs")
    mp.spawn(_tp_train_worker, args=(2, port(), str(run), None), nprocs=2, join=True)
    path = ck.find_latest_checkpoint(str(run / "checkpoints"))
    assert path and ck.read_manifest(path)["tp"] == 2
    cfg = HippoConfig(**DIMS)
    merged_file = str(tmp_path / "merged.pt")
    merged = merge_checkpoint(path, cfg, merged_file)["model_state_dict"]
    shard1 = torch.load(path[:-3] + ".rank1.pt", weights_only=False)["model_state_dict"]
    assert torch.equal(split_plain_state_dict(merged, cfg, 2, 1)["layers.0.attn.qkv_proj.weight"], shard1["layers.0.attn.qkv_proj.weight"])
    m = HippoModel(cfg)
    m.load_state_dict(merged, strict=True)
    served = build_model_and_load(path, cfg, torch.device("cpu"))            # the multi-rank checkpoint itself
    assert all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), served.state_dict().values()))
    # --init_from: one rank and two ranks
    for world in (1, 2):
        rd = tmp_path / f"init{world}"
        os.makedirs(rd / "checkpoints"); os.makedirs(rd / "logs")
        if world == 1:
            for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
                os.environ.pop(k, None)
        mp.spawn(_tp_train_worker, args=(world, port(), str(rd), merged_file), nprocs=world, join=True)
        for r in range(world):
            got = torch.load(rd / f"init_sd.{r}.pt")
            want = split_plain_state_dict(merged, cfg, world, r)
            assert set(got) == set(want) and all(torch.equal(got[k], want[k]) for k in want), (world, r)
