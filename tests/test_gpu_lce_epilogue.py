"""Linear + cross-entropy head with the softmax statistics taken in the logits GEMM epilogue (``lce_epilogue_stats``):
kernels against fp32 torch references, and the whole head against ``F.cross_entropy`` and the fp32-logits path."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


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
