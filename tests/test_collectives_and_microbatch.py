"""Autograd rules of the tensor-parallel collectives (two gloo ranks on the CPU) and micro-batch loss averaging.

* ``gather_seq`` / ``reduce_scatter_seq`` / ``copy_to_tp`` / ``reduce_from_tp``: forward values and the conjugate collective
  in backward (gather <-> reduce-scatter, identity <-> all-reduce), against the same expressions on the concatenated
  tensors in one process (the reference's ``test/test_allgather_grad.py`` checks its all-gather rule the same way).
* A step cut into micro-batches whose numbers of valid targets differ gives the loss and the update of the undivided step:
  every micro-batch loss is weighted by its share of the step's valid targets (``test/test_chunk_loss_averaging.py``)."""
import os

import torch
import torch.multiprocessing as mp

from test_parallel_parity import _args, _batch, _free_port


def _coll_worker(rank, world, port, out_path):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    import torch.distributed as dist
    from hippolm_b200.parallel import collectives as c
    from hippolm_b200.parallel.mesh import init_mesh
    dist.init_process_group("gloo", rank=rank, world_size=world)
    init_mesh(world, 1)
    g = torch.Generator().manual_seed(100 + rank)
    res = {}
    # every rank weighs the outputs differently, so that backward really has something to reduce
    x = torch.randn(6, 5, generator=g, requires_grad=True)
    wgt = torch.randn(6 * world, 5, generator=torch.Generator().manual_seed(7 + rank))
    y = c.gather_seq(x); (y * wgt).sum().backward()
    res["gather"] = (x.detach().clone(), wgt, y.detach().clone(), x.grad.clone())
    x2 = torch.randn(6 * world, 5, generator=g, requires_grad=True)
    w2 = torch.randn(6, 5, generator=torch.Generator().manual_seed(17 + rank))
    y2 = c.reduce_scatter_seq(x2); (y2 * w2).sum().backward()
    res["rs"] = (x2.detach().clone(), w2, y2.detach().clone(), x2.grad.clone())
    x3 = torch.randn(4, 3, generator=g, requires_grad=True)
    w3 = torch.randn(4, 3, generator=torch.Generator().manual_seed(27 + rank))
    y3 = c.copy_to_tp(x3); (y3 * w3).sum().backward()
    res["copy"] = (x3.detach().clone(), w3, y3.detach().clone(), x3.grad.clone())
    x4 = torch.randn(4, 3, generator=g, requires_grad=True)
    w4 = torch.randn(4, 3, generator=torch.Generator().manual_seed(37 + rank))
    y4 = c.reduce_from_tp(x4); (y4 * w4).sum().backward()
    res["reduce"] = (x4.detach().clone(), w4, y4.detach().clone(), x4.grad.clone())
    torch.save(res, out_path + f".{rank}")
    dist.destroy_process_group()


def test_collectives_have_conjugate_backward(tmp_path):
    world, out = 2, str(tmp_path / "coll")
    mp.spawn(_coll_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    r = [torch.load(out + f".{k}") for k in range(world)]
    # all-gather along tokens; backward: every rank gets the sum over ranks of the gradient slice of its own rows
    full = torch.cat([r[k]["gather"][0] for k in range(world)])
    gsum = sum(r[k]["gather"][1] for k in range(world))
    for k in range(world):
        x, w, y, gx = r[k]["gather"]
        assert torch.equal(y, full)
        assert torch.allclose(gx, gsum[6 * k:6 * (k + 1)])
    # reduce-scatter; backward: all-gather of the ranks' output gradients
    tot = sum(r[k]["rs"][0] for k in range(world))
    gfull = torch.cat([r[k]["rs"][1] for k in range(world)])
    for k in range(world):
        x, w, y, gx = r[k]["rs"]
        assert torch.allclose(y, tot[6 * k:6 * (k + 1)])
        assert torch.equal(gx, gfull)
    # identity forward, all-reduce backward (input of a column-parallel region)
    g3 = sum(r[k]["copy"][1] for k in range(world))
    for k in range(world):
        x, w, y, gx = r[k]["copy"]
        assert torch.equal(y, x) and torch.allclose(gx, g3)
    # all-reduce forward, identity backward (output of a row-parallel region)
    s4 = sum(r[k]["reduce"][0] for k in range(world))
    for k in range(world):
        x, w, y, gx = r[k]["reduce"]
        assert torch.allclose(y, s4) and torch.equal(gx, w)


def _one_step(mbs, mask):
    from hippolm_b200.parallel.mesh import init_mesh
    from hippolm_b200.train.loop import setup_worker, teardown_worker, train_step
    init_mesh(1, 1)
    a = _args(1, 1)
    a.micro_batch_size = mbs
    ctx = setup_worker(a, run_dir=None, data_iter=iter(()))
    b = _batch(0, 1)
    labels = b["labels"].clone()
    for s, e in mask:
        labels[s:e] = -100
    out = train_step(ctx, dict(b, labels=labels))
    sd = {k: v.detach().clone() for k, v in ctx.model.state_dict().items()}
    res = float(out["loss"]), float(out["grad_norm"]), sd, labels.numel()
    teardown_worker(ctx)
    return res


def test_micro_batches_with_uneven_valid_targets_average_like_the_whole_step():
    n = _batch(0, 1)["labels"].numel()
    q = n // 4
    # first quarter almost fully masked, third quarter fully masked, the others untouched
    mask = [(8, q), (2 * q, 3 * q)]
    loss_full, gn_full, sd_full, _ = _one_step(0, mask)
    loss_mb, gn_mb, sd_mb, _ = _one_step(q, mask)
    assert abs(loss_full - loss_mb) < 2e-5 * max(1.0, abs(loss_full)), (loss_full, loss_mb)
    assert abs(gn_full - gn_mb) < 1e-3 * gn_full, (gn_full, gn_mb)
    for k in sd_full:
        assert torch.allclose(sd_full[k].float(), sd_mb[k].float(), atol=2e-4, rtol=1e-3), k
    # an unweighted mean of the four micro-batch losses would differ: the masked quarters carry few or no targets
    loss_plain, _, _, _ = _one_step(0, [])
    assert abs(loss_plain - loss_full) > 1e-4
