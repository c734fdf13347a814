"""Muon / AdamW maths, parameter routing, grad-norm clip, host fused kernels, gradient offload."""
import math
import os

import pytest
import torch
import torch.nn as nn

from hippolm_b200.config import HippoConfig
from hippolm_b200.models.model import HippoModel
from hippolm_b200.optim import host_fused
from hippolm_b200.optim.offload import GradOffloader
from hippolm_b200.optim.optimizers import Muon, AdamW, build_param_groups, global_grad_norm, clip_coefficient
from hippolm_b200.ref.ops import newton_schulz5


def _tiny(**kw):
    base = dict(vocab_size=128, hidden_size=32, num_heads=2, head_dim=16, num_layers=4, num_blocks=2, intermediate_size=64)
    base.update(kw)
    return HippoModel(HippoConfig(**base))


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    for shape in ((32, 64), (64, 32)):
        G = torch.randn(*shape)
        X = newton_schulz5(G, 5)
        s = torch.linalg.svdvals(X)
        assert s.max() < 1.3 and s.min() > 0.5


def test_muon_step_matches_formula():
    torch.manual_seed(0)
    p = nn.Parameter(torch.randn(16, 32))
    g = torch.randn(16, 32)
    p.grad = g.clone()
    opt = Muon(lr=0.1, momentum=0.9, weight_decay=0.01, momentum_dtype=torch.float32)
    opt.add_param(p, "w")
    w0 = p.detach().clone()
    opt.step(grad_scale=0.5)
    m = 0.5 * g
    u = 0.5 * g + 0.9 * m
    ref = w0 * (1 - 0.1 * 0.01) - 0.1 * newton_schulz5(u, 5)
    assert torch.allclose(p.detach(), ref, atol=1e-5)
    assert torch.allclose(opt.entries[0].exp_avg, m)


def test_muon_segments_and_row_chunks():
    torch.manual_seed(0)
    p = nn.Parameter(torch.randn(24, 16))
    p.muon_segments = [(0, 8), (8, 24)]
    p.grad = torch.randn(24, 16)
    opt = Muon(lr=1.0, momentum=0.0, momentum_dtype=torch.float32)
    opt.add_param(p, "w")
    w0, g = p.detach().clone(), p.grad.clone()
    opt.step()
    ref = torch.cat([newton_schulz5(g[:8], 5), newton_schulz5(g[8:], 5)])
    assert torch.allclose(w0 - p.detach(), ref, atol=1e-5)
    opt2 = Muon(lr=1.0, momentum=0.0, ns_row_chunk=4)
    assert opt2._segments(type("E", (), {"shape": (10, 4), "param": None})()) == [(0, 4), (4, 8), (8, 10)]


def test_adamw_standard_and_reference_compat():
    torch.manual_seed(0)
    for compat in (False, True):
        p = nn.Parameter(torch.randn(50)); g = torch.randn(50); p.grad = g.clone()
        opt = AdamW(lr=0.01, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, m_dtype=torch.float32,
                    v_dtype=torch.float32, reference_compat=compat)
        opt.add_param(p, "p")
        w0 = p.detach().clone()
        opt.step()
        m = 0.1 * g
        if compat:
            v = 0.05 * m * m
            upd = m / ((v / 0.05).sqrt() + 1e-8)
        else:
            v = 0.05 * g * g
            upd = (m / 0.1) / ((v / 0.05).sqrt() + 1e-8)
        assert torch.allclose(p.detach(), w0 * (1 - 0.001) - 0.01 * upd, atol=1e-6)


def test_param_routing():
    model = _tiny(ffn_nvfp4=True, ffn_nvfp4_no_bf16_master=True)
    muon, adamw = build_param_groups(model)
    mnames = {e.name for e in muon.entries}
    anames = {e.name for e in adamw.entries}
    assert "embed_tokens.weight" in anames and "lm_head.weight" in anames and "norm.weight" in anames
    assert "attn_res.query" in anames and "layers.0.attn.A_log" in anames and "layers.0.attn.g_proj1_bias" in anames
    assert "layers.0.attn.in_proj_weight" in mnames and "layers.3.attn.qkv_proj_weight" in mnames
    assert "layers.0.ffn.gate_up_proj" in mnames and "layers.0.ffn.down_proj" in mnames     # NVFP4 modules
    assert sum(e.param is None for e in muon.entries) == 8


def test_grad_norm_and_clip():
    model = _tiny()
    muon, adamw = build_param_groups(model)
    tot = 0.0
    for p in model.parameters():
        p.grad = torch.randn_like(p)
        tot += float(p.grad.float().pow(2).sum())
    n = float(global_grad_norm(muon, adamw))
    assert abs(n - math.sqrt(tot)) < 1e-3 * math.sqrt(tot)
    assert clip_coefficient(0.5, 1.0) == 1.0
    assert clip_coefficient(4.0, 1.0) == pytest.approx(1.0 / (4.0 + 1e-6))
    assert clip_coefficient(float("nan"), 1.0) == 1.0


def test_optimizer_state_dict_roundtrip():
    model = _tiny()
    muon, adamw = build_param_groups(model)
    for p in model.parameters():
        p.grad = torch.randn_like(p)
    muon.step(); adamw.step()
    sd_m, sd_a = muon.state_dict(), adamw.state_dict()
    assert {"lr", "momentum", "weight_decay", "nesterov", "ns_steps", "state"} <= set(sd_m)
    assert {"shape", "step", "kind", "grad", "exp_avg"} <= set(sd_m["state"][0])
    assert {"exp_avg", "exp_avg_sq"} <= set(sd_a["state"][0])
    muon2, adamw2 = build_param_groups(_tiny())
    muon2.load_state_dict(sd_m); adamw2.load_state_dict(sd_a)
    assert torch.equal(muon2.entries[3].exp_avg, muon.entries[3].exp_avg) and adamw2.entries[0].step == 1
    sd_m["state"].pop()
    with pytest.raises(ValueError):
        muon2.load_state_dict(sd_m)


@pytest.mark.parametrize("force_py", ["0", "1"])
def test_host_fused_kernels(force_py, monkeypatch):
    monkeypatch.setenv("HIPPO_FUSED_FORCE_PYLOOP", force_py)
    torch.manual_seed(0)
    a = [torch.randn(1000).bfloat16(), torch.randn(77)]
    b = [torch.randn(1000).bfloat16(), torch.randn(77).bfloat16()]
    ref = [(x.float() + y.float()) for x, y in zip(a, b)]
    host_fused.fused_add_into_many(a, b)
    assert torch.allclose(a[0].float(), ref[0].bfloat16().float()) and torch.allclose(a[1], ref[1])
    n2 = host_fused.fused_l2_norm_sq(a)
    assert abs(n2 - sum(float(t.double().pow(2).sum()) for t in a)) < 1e-3 * n2
    assert host_fused.fused_inf_nan_count(a) == 0
    a[1][3] = float("nan"); a[0][5] = float("inf")
    assert host_fused.fused_inf_nan_count(a) == 2
    a[1][3] = 1.0; a[0][5] = 1.0
    c = a[1].clone()
    host_fused.fused_scale_many(a, 0.5)
    assert torch.allclose(a[1], c * 0.5)
    host_fused.fused_zero_many(a)
    assert float(a[0].float().abs().sum()) == 0 and float(a[1].abs().sum()) == 0
    g, m, v = torch.randn(300), torch.zeros(300), torch.zeros(300)
    g0 = g.clone()
    host_fused.fused_adam_step(g, m, v, 0.9, 0.95, 1e-8, 1)
    assert torch.allclose(m, 0.1 * g0, atol=1e-6) and torch.allclose(v, 0.05 * g0 * g0, atol=1e-6)
    assert torch.allclose(g, g0.sign(), atol=1e-3)


_ISA_CHILD = r'''
import os, sys, torch
sys.path.insert(0, os.environ["HIPPO_ROOT"])
from hippolm_b200.optim import host_fused as hf
want = os.environ.get("HIPPO_HOST_ISA", "")
assert hf.isa() in ("avx512", "avx2")
if want == "avx2":
    assert hf.isa() == "avx2"
torch.manual_seed(0)
n = 200003                                            # several OpenMP blocks and a ragged tail
for dd in (torch.float32, torch.bfloat16):
    for sd in (torch.float32, torch.bfloat16):
        d = (3 * torch.randn(n)).to(dd); s = torch.randn(n).to(sd)
        d[7] = float("nan"); s[11] = float("inf")
        ref = (d.float() + s.float()).to(dd)          # torch narrows with round-to-nearest-even as well
        hf.fused_add_into_many([d], [s])
        same = (d.view(torch.int16) == ref.view(torch.int16)) if dd == torch.bfloat16 else (d == ref)
        nan_ok = torch.isnan(d) & torch.isnan(ref)
        assert bool((same | nan_ok).all()), (dd, sd)
    t = torch.randn(n).to(dd)
    ref = (t.float() * 0.37).to(dd); hf.fused_scale_many([t], 0.37)
    assert torch.equal(t, ref)
    exact = float(t.double().pow(2).sum())
    assert abs(hf.fused_l2_norm_sq([t]) - exact) < 1e-9 * exact
    t[5] = float("inf"); t[n - 1] = float("nan"); t[40000] = -float("inf")
    assert hf.fused_inf_nan_count([t]) == 3
for gd, md, vd in ((torch.float32,) * 3, (torch.bfloat16,) * 3, (torch.bfloat16, torch.float32, torch.float32)):
    for compat in (False, True):
        g = torch.randn(n).to(gd); m = (0.1 * torch.randn(n)).to(md); v = (0.01 * torch.rand(n)).to(vd)
        g0, m0, v0 = g.float().clone(), m.float().clone(), v.float().clone()
        hf.fused_adam_step(g, m, v, 0.9, 0.95, 1e-8, 3, grad_scale=0.5, reference_compat=compat)
        gs = g0 * 0.5
        mr = 0.9 * m0 + 0.1 * gs
        vr = 0.95 * v0 + 0.05 * (mr * mr if compat else gs * gs)
        bc1, bc2 = 1 - 0.9 ** 3, 1 - 0.95 ** 3
        ur = mr / ((vr / bc2).sqrt() + 1e-8) if compat else (mr / bc1) / ((vr / bc2).sqrt() + 1e-8)
        tol = 1e-5 if gd == torch.float32 else 1e-2
        assert torch.allclose(m.float(), mr.to(md).float(), rtol=tol, atol=tol)
        assert torch.allclose(v.float(), vr.to(vd).float(), rtol=tol, atol=tol)
        assert torch.allclose(g.float(), ur, rtol=max(tol, 2e-2 if md == torch.bfloat16 else tol), atol=tol), (gd, md, vd, compat)
print("HOST_OK", hf.isa())
'''


@pytest.mark.parametrize("force_isa", ["", "avx2"])
def test_host_kernels_both_instruction_sets(force_isa, tmp_path):
    """The CPUID-dispatched host kernels (AVX-512 build where the CPU has it, AVX2 build otherwise or when forced):
    bf16 round-to-nearest-even bit for bit against torch, NaN / inf handling, every dtype combination of the AdamW step."""
    import subprocess
    import sys
    if host_fused.isa() == "python":
        pytest.skip("host library not built")
    script = tmp_path / "child.py"
    script.write_text(_ISA_CHILD)
    env = dict(os.environ, HIPPO_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env.pop("HIPPO_FUSED_FORCE_PYLOOP", None)
    if force_isa:
        env["HIPPO_HOST_ISA"] = force_isa
    r = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "HOST_OK" in r.stdout, r.stdout[-1500:] + r.stderr[-3000:]


@pytest.mark.parametrize("async_worker", [True, False])
def test_grad_offload_accumulates_and_frees(async_worker):
    torch.manual_seed(0)
    lin = nn.Linear(8, 4)
    off = GradOffloader(lin, torch.device("cpu"), accum_dtype=torch.float32, async_worker=async_worker)
    x = torch.randn(5, 8)
    total = {n: torch.zeros_like(p) for n, p in lin.named_parameters()}
    for _ in range(3):
        ref = nn.Linear(8, 4); ref.load_state_dict(lin.state_dict())
        ref(x).sum().backward()
        for n, p in ref.named_parameters():
            total[n] += p.grad
        lin(x).sum().backward()
        assert all(p.grad is None for p in lin.parameters())       # freed by the hook
        off.after_microbatch()
    assert off.drain(5.0)
    for n, p in lin.named_parameters():
        assert torch.allclose(off.accum[id(p)], total[n], atol=1e-5)
    off.drain_to_device()
    for n, p in lin.named_parameters():
        assert torch.allclose(p.grad, total[n], atol=1e-5)
    assert all(float(a.abs().sum()) == 0 for a in off.host_grads())
    off.close(); off.close()


def test_grad_offload_manual_flush():
    lin = nn.Linear(4, 4, bias=False)
    off = GradOffloader(lin, torch.device("cpu"), accum_dtype=torch.float32, async_worker=False,
                        manual_flush=[lin.weight])
    lin(torch.ones(2, 4)).sum().backward()
    assert lin.weight.grad is not None                             # not touched by a hook
    off.after_microbatch()
    assert lin.weight.grad is None and float(off.accum[id(lin.weight)].sum()) == 32.0
    off.close()
