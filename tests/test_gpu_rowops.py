"""Row kernels vs fp32 torch references (forward and backward)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err <= tol * scale, f"max err {err} vs scale {scale}"


@pytest.mark.parametrize("T,D", [(64, 256), (333, 4096), (1000, 2048)])
def test_rmsnorm(T, D):
    from hippolm_b200 import ops
    from hippolm_b200.ref import ops as ro
    x = torch.randn(T, D, device="cuda").bfloat16().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16().requires_grad_(True)
    dy = torch.randn(T, D, device="cuda").bfloat16()
    y = ops.rmsnorm(x, w, 1e-6)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = ro.rmsnorm(xr, wr, 1e-6)
    yr.backward(dy.float())
    _close(y, yr, 1e-2); _close(x.grad, xr.grad, 2e-2); _close(w.grad, wr.grad, 2e-2)


def test_gated_rmsnorm_and_swiglu():
    from hippolm_b200 import ops
    from hippolm_b200.ref import kda as rk, ops as ro
    T, H, V = 257, 4, 128
    o = torch.randn(T, H, V, device="cuda").bfloat16().requires_grad_(True)
    g = torch.randn(T, H, V, device="cuda").bfloat16().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(V, device="cuda")).bfloat16().requires_grad_(True)
    dy = torch.randn(T, H, V, device="cuda").bfloat16()
    y = ops.gated_rmsnorm(o, g, w, 1e-6); y.backward(dy)
    o2, g2, w2 = (t.detach().float().requires_grad_(True) for t in (o, g, w))
    y2 = rk.gated_rmsnorm(o2, g2, w2, 1e-6); y2.backward(dy.float())
    _close(y, y2, 1e-2); _close(o.grad, o2.grad, 2e-2); _close(g.grad, g2.grad, 2e-2); _close(w.grad, w2.grad, 2e-2)
    gu = torch.randn(T, 512, device="cuda").bfloat16().requires_grad_(True)
    da = torch.randn(T, 256, device="cuda").bfloat16()
    a = ops.swiglu(gu); a.backward(da)
    gu2 = gu.detach().float().requires_grad_(True)
    a2 = ro.swiglu(gu2); a2.backward(da.float())
    _close(a, a2, 1e-2); _close(gu.grad, gu2.grad, 2e-2)


@pytest.mark.parametrize("safe", [False, True])
def test_kda_gate(safe):
    from hippolm_b200 import ops
    from hippolm_b200.ref import kda as rk
    T, H, K = 200, 4, 128
    x = torch.randn(T, H, K, device="cuda").bfloat16().requires_grad_(True)
    A = torch.randn(H, device="cuda").mul(0.5).requires_grad_(True)
    b = torch.randn(H * K, device="cuda").mul(0.5).requires_grad_(True)
    dg = torch.randn(T, H, K, device="cuda")
    g = ops.kda_gate(x, A, b, safe, -5.0); g.backward(dg)
    x2, A2, b2 = (t.detach().float().requires_grad_(True) for t in (x, A, b))
    g2 = rk.kda_gate(x2, A2, b2, safe, -5.0); g2.backward(dg)
    _close(g, g2, 1e-3); _close(x.grad, x2.grad, 2e-2); _close(A.grad, A2.grad, 2e-2); _close(b.grad, b2.grad, 2e-2)


def test_rope():
    from hippolm_b200 import ops
    from hippolm_b200.ref import ops as ro
    T, H, dh = 300, 4, 128
    q = torch.randn(T, H, dh, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(T, H, dh, device="cuda").bfloat16()
    pos = torch.arange(T, device="cuda") % 97
    q1, k1 = ops.rope(q, k, pos, 10000.0)
    cos, sin = ro.rope_tables(pos, dh, 10000.0)
    _close(q1, ro.apply_rope(q.detach().float(), cos, sin), 1e-2)
    _close(k1, ro.apply_rope(k.float(), cos, sin), 1e-2)
    dq = torch.randn_like(q1)
    q1.backward(dq)
    qf = q.detach().float().requires_grad_(True)
    ro.apply_rope(qf, cos, sin).backward(dq.float())
    _close(q.grad, qf.grad, 1e-2)


def test_short_conv_silu_varlen():
    from hippolm_b200 import ops
    from hippolm_b200.ref import kda as rk
    T, D, W = 300, 256, 4
    proj = torch.randn(T, 3 * D, device="cuda").bfloat16()
    x = proj[:, D:2 * D].detach().requires_grad_(True)          # strided view, as in the model
    w = (0.5 * torch.randn(D, W, device="cuda")).bfloat16().requires_grad_(True)
    cu = torch.tensor([0, 1, 50, 51, 52, 300], dtype=torch.int32, device="cuda")
    dy = torch.randn(T, D, device="cuda").bfloat16()
    y = ops.short_conv_silu(x, w, None, cu); y.backward(dy)
    x2, w2 = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    y2 = rk.short_conv_silu(x2, w2, None, cu); y2.backward(dy.float())
    _close(y, y2, 1e-2); _close(x.grad, x2.grad, 2e-2); _close(w.grad, w2.grad, 2e-2)


@pytest.mark.parametrize("T,D", [(333, 4096), (64, 256)])
def test_add_rmsnorm_matches_add_then_norm(T, D):
    """Residual add fused into the norm behind it: both results and all three gradients (the sum is consumed twice, once
    by the norm and once by whatever follows on the residual path) against the unfused fp32 composition."""
    from hippolm_b200 import ops
    from hippolm_b200.ref import ops as ro
    torch.manual_seed(T)
    x = torch.randn(T, D, device="cuda").bfloat16().requires_grad_(True)
    r = torch.randn(T, D, device="cuda").bfloat16().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16().requires_grad_(True)
    ds, dy = torch.randn(T, D, device="cuda").bfloat16(), torch.randn(T, D, device="cuda").bfloat16()
    s, y = ops.add_rmsnorm(x, r, w, 1e-6)
    torch.autograd.backward([s, y], [ds, dy])
    xr, rr, wr = (t.detach().float().requires_grad_(True) for t in (x, r, w))
    sr = xr + rr
    yr = ro.rmsnorm(sr, wr, 1e-6)
    torch.autograd.backward([sr, yr], [ds.float(), dy.float()])
    _close(s, sr, 1e-2); _close(y, yr, 1e-2)
    _close(x.grad, xr.grad, 2e-2); _close(r.grad, rr.grad, 2e-2); _close(w.grad, wr.grad, 2e-2)
    assert torch.equal(x.grad, r.grad)
    # only the norm output used: the residual-path gradient is absent
    x2 = x.detach().clone().requires_grad_(True)
    _, y2 = ops.add_rmsnorm(x2, r.detach(), w.detach(), 1e-6)
    y2.backward(dy)
    x3 = x.detach().float().requires_grad_(True)
    ro.rmsnorm(x3 + r.detach().float(), w.detach().float(), 1e-6).backward(dy.float())
    _close(x2.grad, x3.grad, 2e-2)


def test_kda_prologue_gate_columns_pass_through():
    """The low-rank gate inputs leave the prologue as a contiguous copy and their gradient comes back through it into the
    one projection gradient (padding columns zero), like slicing the projection would."""
    from hippolm_b200 import ops
    torch.manual_seed(3)
    T, H, K = 200, 4, 128
    key = H * K
    o_fg, fgw = 3 * key, 2 * K
    n = o_fg + fgw + H + 28                                       # 28 padding columns
    proj = (0.5 * torch.randn(T, n, device="cuda")).bfloat16().requires_grad_(True)
    q, k, v, beta, fg = ops.kda_prologue(proj, H, K, 0, key, 2 * key, o_fg + fgw, K ** -0.5, 2.0, True, o_fg, fgw)
    assert fg.is_contiguous() and torch.equal(fg, proj.detach()[:, o_fg:o_fg + fgw])
    gs = [torch.randn_like(t.float()).to(t.dtype) for t in (q, k, v, beta, fg)]
    torch.autograd.backward([q, k, v, beta, fg], gs)
    pc = proj.detach().cpu().float().requires_grad_(True)
    outs = ops.kda_prologue(pc, H, K, 0, key, 2 * key, o_fg + fgw, K ** -0.5, 2.0, True, o_fg, fgw)
    torch.autograd.backward(list(outs), [g.cpu().float() for g in gs])
    for a, b in zip((q, k, v, beta), outs[:4]):
        _close(a.cpu(), b, 2e-2)
    _close(proj.grad.cpu(), pc.grad, 3e-2)
    assert float(proj.grad[:, o_fg + fgw + H:].abs().max()) == 0.0
    assert torch.equal(proj.grad[:, o_fg:o_fg + fgw], gs[4])
