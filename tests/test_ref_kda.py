"""The chunked torch KDA must reproduce the token recurrence (forward, final state, varlen, h0)."""
import torch
import pytest

from hippolm_b200.ref.kda import kda_recurrent, kda_chunked, l2norm, kda_gate


def _inputs(T, H, K, V, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    q = l2norm(torch.randn(T, H, K, generator=g))
    k = l2norm(torch.randn(T, H, K, generator=g))
    v = torch.randn(T, H, V, generator=g)
    gd = -torch.nn.functional.softplus(torch.randn(T, H, K, generator=g))
    beta = torch.sigmoid(torch.randn(T, H, generator=g))
    return [t.to(dtype) for t in (q, k, v, gd, beta)]


@pytest.mark.parametrize("T,cu", [(96, None), (200, [0, 37, 101, 165, 200]), (64, [0, 64])])
def test_chunked_matches_recurrent(T, cu):
    q, k, v, g, beta = _inputs(T, 2, 16, 24)
    cu_t = torch.tensor(cu) if cu is not None else None
    N = (len(cu) - 1) if cu is not None else 1
    h0 = torch.randn(N, 2, 16, 24) * 0.1
    o1, s1 = kda_recurrent(q, k, v, g, beta, initial_state=h0, cu_seqlens=cu_t)
    o2, s2 = kda_chunked(q, k, v, g, beta, initial_state=h0, cu_seqlens=cu_t, chunk=32)
    assert torch.allclose(o1, o2, atol=2e-5, rtol=1e-4)
    assert torch.allclose(s1, s2, atol=2e-5, rtol=1e-4)


def test_chunked_gradients_match_recurrent():
    q, k, v, g, beta = _inputs(70, 2, 8, 8, seed=3, dtype=torch.float64)
    cu = torch.tensor([0, 30, 70])
    outs = []
    for fn in (kda_recurrent, kda_chunked):
        ins = [t.clone().requires_grad_(True) for t in (q, k, v, g, beta)]
        o, s = fn(*ins, cu_seqlens=cu)
        (o.square().sum() + s.sum()).backward()
        outs.append([t.grad for t in ins])
    for a, b in zip(*outs):
        assert torch.allclose(a, b, atol=1e-4, rtol=1e-3)


def test_state_resets_at_boundaries():
    q, k, v, g, beta = _inputs(80, 1, 8, 8, seed=5)
    cu = torch.tensor([0, 40, 80])
    o, _ = kda_chunked(q, k, v, g, beta, cu_seqlens=cu, chunk=16)
    o2, _ = kda_chunked(q[40:], k[40:], v[40:], g[40:], beta[40:], chunk=16)
    assert torch.allclose(o[40:], o2, atol=1e-5)


def test_gate_forms():
    x = torch.randn(5, 2, 4)
    A = torch.zeros(2)
    b = torch.zeros(8)
    g = kda_gate(x, A, b, safe_gate=True, lower_bound=-5.0)
    assert (g <= 0).all() and (g >= -5).all()
    g2 = kda_gate(x, A, b, safe_gate=False)
    assert torch.allclose(g2, -torch.nn.functional.softplus(x))


def test_anchored_matches_recurrent_strong_decay():
    from hippolm_b200.ref.kda import kda_chunked_anchored
    q, k, v, g, beta = _inputs(150, 2, 16, 16, seed=7)
    g = g * 12.0          # decay far beyond what a one-sided factorisation survives in fp32
    cu = torch.tensor([0, 70, 150])
    o1, s1 = kda_recurrent(q, k, v, g, beta, cu_seqlens=cu)
    o2, s2 = kda_chunked_anchored(q, k, v, g, beta, cu_seqlens=cu)
    assert torch.isfinite(o2).all()
    assert torch.allclose(o1, o2, atol=2e-5, rtol=1e-4)
    assert torch.allclose(s1, s2, atol=2e-5, rtol=1e-4)
