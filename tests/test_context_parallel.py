"""KDA context parallelism (CPU, gloo, 2 ranks): a sequence split in two segments reproduces the single-device
outputs, final state and input gradients."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _inputs(T, H, K, V):
    g = torch.Generator().manual_seed(5)
    q = torch.randn(T, H, K, generator=g); k = torch.randn(T, H, K, generator=g); v = torch.randn(T, H, V, generator=g)
    gd = -torch.nn.functional.softplus(torch.randn(T, H, K, generator=g))
    beta = torch.sigmoid(torch.randn(T, H, generator=g))
    wo = torch.randn(T, H, V, generator=g)
    return q, k, v, gd, beta, wo


def _run(rank, world, port, out_path):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from hippolm_b200 import ops
    from hippolm_b200.parallel.context import kda_context_parallel
    T, H, K, V = 192, 2, 16, 16
    full = [t.clone().requires_grad_(True) for t in _inputs(T, H, K, V)[:5]]
    wo = _inputs(T, H, K, V)[5]
    o_ref, s_ref = ops.kda(*full)
    ((o_ref * wo).sum() + s_ref.sum()).backward()
    seg = T // world
    sl = slice(rank * seg, (rank + 1) * seg)
    loc = [t.detach()[sl].clone().requires_grad_(True) for t in full]
    o, s_fin = kda_context_parallel(*loc, group=dist.group.WORLD)
    # the final state is the same tensor on every rank: count its loss term once (rank 0), the gather's backward sums
    loss = (o * wo[sl]).sum() + (s_fin.sum() if rank == 0 else 0.0 * s_fin.sum())
    loss.backward()
    err_o = (o - o_ref.detach()[sl]).abs().max().item()
    err_s = (s_fin - s_ref.detach()).abs().max().item()
    err_g = max((a.grad - b.grad[sl]).abs().max().item() for a, b in zip(loc, full))
    torch.save({"err_o": err_o, "err_s": err_s, "err_g": err_g}, out_path + f".{rank}")
    dist.destroy_process_group()


def test_kda_context_parallel_matches_single_device(tmp_path):
    out = str(tmp_path / "cp")
    mp.spawn(_run, args=(2, _free_port(), out), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(out + f".{r}")
        assert res["err_o"] < 2e-4, res
        assert res["err_s"] < 2e-4, res
        assert res["err_g"] < 2e-3, res
