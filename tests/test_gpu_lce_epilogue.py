"""Linear + cross-entropy head with the softmax statistics taken in the logits GEMM epilogue (``lce_epilogue_stats``):
kernels against fp32 torch references, and the whole head against ``F.cross_entropy`` and the fp32-logits path."""
import os
import socket
import subprocess
import sys

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()


def _cos(a, b):
    return F.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()


@pytest.mark.parametrize("C,D,V", [(300, 256, 1000), (1024, 512, 16032), (130, 128, 256), (257, 64, 264)])
def test_logits_gemm_epilogue_statistics(C, D, V):
    """bf16 logits, per-tile (max, sum exp) merged per row, target logit: against x @ w^T in fp32 rounded to bf16."""
    from hippolm_b200.ops import cuda_ops as co
    torch.manual_seed(C + V)
    x = torch.randn(C, D, device="cuda").bfloat16()
    w = (0.2 * torch.randn(V, D, device="cuda")).bfloat16()
    tg = torch.randint(0, V, (C,), device="cuda")
    tg[::7] = -1
    tg[1] = V - 1
    tg[2] = 0
    z, part, tz, tg64 = co.lce_logits_stats(x, w, tg)
    zr = (x.float() @ w.float().t())
    assert z.dtype == torch.bfloat16 and _rel(z, zr) < 1e-2
    # the statistics describe the STORED logits exactly (up to fp32 summation order)
    zs = z.float()
    p = part.view(-1, C, 2)
    assert p.shape[0] == (V + 255) // 256
    for t in range(p.shape[0]):
        cols = zs[:, t * 256:min(V, (t + 1) * 256)]
        assert torch.equal(p[t, :, 0], cols.max(-1).values)
        assert _rel(p[t, :, 1], (cols - cols.max(-1, keepdim=True).values).exp().sum(-1)) < 1e-4
    rows = (tg >= 0).nonzero(as_tuple=True)[0]
    assert torch.equal(tz[rows], zs[rows, tg[rows]])
    # merge + gradient in place
    roww = (tg >= 0).float() / 10.0
    loss_sum = torch.zeros(1, device="cuda")
    ref = torch.softmax(zs, -1)
    ref[rows, tg[rows]] -= 1
    ref = ref * roww.unsqueeze(-1)
    loss_ref = (torch.logsumexp(zs[rows], -1) - zs[rows, tg[rows]]).sum()
    dz = co.lce_grad_inplace_local(z, part, tz, tg64, roww, loss_sum)
    assert dz.data_ptr() == z.data_ptr()
    assert (dz.float() - ref).abs().max() < 1e-3
    assert abs(loss_sum.item() - loss_ref.item()) < 1e-3 * max(1.0, abs(loss_ref.item()))


def _head_loss(epi, x, w, targets, chunks):
    from hippolm_b200.models.model import _VocabParallelLCE
    x = x.clone().requires_grad_(True)
    w = w.clone().requires_grad_(True)
    nv = int((targets >= 0).sum())
    loss = _VocabParallelLCE.apply(x, w, targets, 0, chunks, nv, epi)
    loss.backward()
    return loss.detach(), x.grad, w.grad


@pytest.mark.parametrize("T,D,V,chunks", [(512, 256, 128256, 0), (700, 512, 4096, 3)])
def test_head_with_epilogue_statistics_matches_cross_entropy(T, D, V, chunks):
    from hippolm_b200.parallel.mesh import init_mesh
    init_mesh(1, 1)
    torch.manual_seed(T)
    x = torch.randn(T, D, device="cuda").bfloat16()
    w = (0.05 * torch.randn(V, D, device="cuda")).bfloat16()
    targets = torch.randint(0, V, (T,), device="cuda")
    targets[::5] = -100
    loss_e, dx_e, dw_e = _head_loss(True, x, w, targets, chunks)
    loss_f, dx_f, dw_f = _head_loss(False, x, w, targets, chunks)
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    loss_r = F.cross_entropy(xr @ wr.t(), targets, ignore_index=-100)
    loss_r.backward()
    assert abs(loss_e.item() - loss_r.item()) < 2e-3 * abs(loss_r.item())
    assert abs(loss_e.item() - loss_f.item()) < 2e-3 * abs(loss_r.item())
    assert _cos(dx_e, xr.grad) > 0.999 and _cos(dw_e, wr.grad) > 0.999
    assert _rel(dx_e, xr.grad) < 3e-2 and _rel(dw_e, wr.grad) < 3e-2
    assert _cos(dx_e, dx_f) > 0.999 and _cos(dw_e, dw_f) > 0.999


def test_epilogue_path_keeps_fp32_logits_out_of_memory():
    """The chunk's logits exist only as bf16: peak memory of the head drops by about the size of the fp32 tile."""
    from hippolm_b200.parallel.mesh import init_mesh
    init_mesh(1, 1)
    T, D, V = 2048, 256, 65536
    torch.manual_seed(0)
    x = torch.randn(T, D, device="cuda").bfloat16()
    w = (0.05 * torch.randn(V, D, device="cuda")).bfloat16()
    targets = torch.randint(0, V, (T,), device="cuda")
    peaks = []
    for epi in (False, True):
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        base = torch.cuda.memory_allocated()
        _head_loss(epi, x, w, targets, 1)
        torch.cuda.synchronize()
        peaks.append(torch.cuda.max_memory_allocated() - base)
    fp32_tile = T * V * 4
    assert peaks[0] - peaks[1] > 0.9 * fp32_tile, peaks


_CHILD = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["HIPPO_ROOT"])
from hippolm_b200.parallel.mesh import init_distributed_from_env, init_mesh
from hippolm_b200.parallel import fused
from hippolm_b200.ops import cuda_ops
from hippolm_b200.models.model import _VocabParallelLCE
dev = init_distributed_from_env()
mesh = init_mesh(tp=dist.get_world_size(), device=dev)
w_, r_ = mesh.tp, mesh.tp_rank
assert fused.setup(mesh, 4096, 4096)
ws = fused._STATE["ws"]
torch.manual_seed(1 + r_)
for it in range(3):
    # kernels: epilogue statistics of this rank's vocabulary shard, merged and pushed, gradient over the logits
    Cr, Vl, De = 256 + 64 * it, 1000, 256
    tgt = torch.randint(0, Vl * w_, (Cr,), device=dev); dist.broadcast(tgt, 0)
    tgt[::7] = -100
    local = tgt - r_ * Vl
    own = (local >= 0) & (local < Vl) & (tgt >= 0)
    local_t = torch.where(own, local, torch.full_like(local, -1))
    valid = tgt >= 0
    roww = valid.float() / valid.sum()
    xe = torch.randn(Cr, De, device=dev).bfloat16(); dist.broadcast(xe, 0)
    We = (0.2 * torch.randn(Vl, De, device=dev)).bfloat16()
    ze, part, tze, tg64 = cuda_ops.lce_logits_stats(xe, We, local_t)
    zs = [torch.empty_like(ze) for _ in range(w_)]
    dist.all_gather(zs, ze, group=mesh.tp_group)
    zfull = torch.cat(zs, 1).float()
    loss_raw = torch.zeros(1, device=dev)
    dze = ws.lce_grad_inplace(ws.lce_part_push(part, tze, tg64), ze, roww, loss_raw)
    lse = torch.logsumexp(zfull, 1)
    tz = zfull.gather(1, tgt.clamp(min=0)[:, None])[:, 0]
    ref_loss = ((lse - tz) * valid).sum()
    assert abs(loss_raw.item() - ref_loss.item()) < 2e-3 * abs(ref_loss.item()), (loss_raw.item(), ref_loss.item())
    pr = (zfull - lse[:, None]).exp()
    pr[valid, tgt[valid]] -= 1
    refdz = (pr * roww[:, None])[:, r_ * Vl:(r_ + 1) * Vl]
    assert (dze.float() - refdz).abs().max() < 2e-2 * roww.max(), "epilogue-statistics CE gradient"
    # whole head, sequence-parallel input shard, both statistics paths on the same data
    Ts, D, V = 384, 256, 2048 * w_
    torch.manual_seed(100 + it)
    xf = torch.randn(Ts * w_, D, device=dev).bfloat16()
    wf = (0.05 * torch.randn(V, D, device=dev)).bfloat16()
    tf = torch.randint(0, V, (Ts * w_,), device=dev); tf[::5] = -100
    nv = int((tf >= 0).sum())
    outs = []
    for epi in (True, False):
        xi = xf[r_ * Ts:(r_ + 1) * Ts].clone().requires_grad_(True)
        wi = wf[r_ * (V // w_):(r_ + 1) * (V // w_)].clone().requires_grad_(True)
        loss = _VocabParallelLCE.apply(xi, wi, tf, r_ * (V // w_), 2, nv, epi)
        loss.backward()
        outs.append((loss.detach().float(), xi.grad.float(), wi.grad.float()))
    xr = xf.float().requires_grad_(True); wr = wf.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(xr @ wr.t(), tf, ignore_index=-100)
    ref.backward()
    gx = xr.grad[r_ * Ts:(r_ + 1) * Ts]; gw = wr.grad[r_ * (V // w_):(r_ + 1) * (V // w_)]
    cos = lambda a, b: torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    for loss, dx, dw in outs:
        assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item()), (loss.item(), ref.item())
        assert cos(dx, gx) > 0.999 and cos(dw, gw) > 0.999, (cos(dx, gx), cos(dw, gw))
    torch.manual_seed(1 + r_ + 10 * it)
torch.cuda.synchronize()
ws.check_status()
dist.barrier()
if r_ == 0: print("LCE_EPILOGUE_OK")
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_epilogue_statistics_two_gpus(tmp_path):
    """Vocabulary-parallel head over two ranks: the merged statistics travel by peer stores, the gradient kernel waits
    (bounded) for both sources; kernels against fp32 references, whole head against F.cross_entropy."""
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    env = dict(os.environ, HIPPO_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "LCE_EPILOGUE_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
