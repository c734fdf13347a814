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
