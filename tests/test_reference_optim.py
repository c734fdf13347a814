"""Optimizer updates against the reference's own classes (``src/training/param_offload/adamw.py``, ``muon.py``) run on the
CPU from the unmodified tree in a child process: AdamW in its compatibility mode (second moment from the first moment, no
first-moment bias correction) and Muon (momentum, Nesterov, five Newton-Schulz steps, decoupled decay) over several steps
with the same gradients. Needs the copy of the reference tree under ``baseline/_ref`` (skipped without it)."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src")), reason="no copy of the reference tree")
def test_optimizer_updates_follow_the_reference(tmp_path):
    from hippolm_b200.optim.optimizers import AdamW, Muon
    from hippolm_b200.parallel.mesh import init_mesh
    init_mesh(1, 1)
    torch.manual_seed(3)
    hyper = dict(lr=1e-2, b1=0.9, b2=0.95, eps=1e-8, wd=0.01, muon_lr=0.02, momentum=0.95, muon_wd=0.1)
    a_shapes, m_shapes, steps = [(64,), (48, 3), (1000, 16)], [(64, 32), (32, 96), (128, 128)], 4
    case = {"hyper": hyper,
            "adamw_params": [torch.randn(s) for s in a_shapes], "muon_params": [0.1 * torch.randn(s) for s in m_shapes],
            "adamw_grads": [[0.01 * (i + 1) * torch.randn(s) for s in a_shapes] for i in range(steps)],
            "muon_grads": [[0.01 * torch.randn(s) for s in m_shapes] for _ in range(steps)]}
    inp, out = str(tmp_path / "case.pt"), str(tmp_path / "ref.pt")
    torch.save(case, inp)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "reference_optim_worker.py"), REF, inp, out],
                       capture_output=True, text=True, timeout=900, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-3000:]
    ref = torch.load(out)

    pa = [torch.nn.Parameter(t.clone()) for t in case["adamw_params"]]
    opt = AdamW(lr=hyper["lr"], betas=(hyper["b1"], hyper["b2"]), eps=hyper["eps"], weight_decay=hyper["wd"],
                m_dtype=torch.float32, v_dtype=torch.float32, reference_compat=True)
    for p in pa:
        opt.add_param(p)
    for i, grads in enumerate(case["adamw_grads"]):
        for p, g in zip(pa, grads):
            p.grad = g.clone()
        opt.step()
        for p, want, start in zip(pa, ref["adamw"][i], case["adamw_params"]):
            moved = (want - start).abs().max()
            assert moved > 0                                          # the reference did update
            assert (p.detach() - want).abs().max() <= 2e-3 * moved + 1e-7, (i, tuple(p.shape))

    pm = [torch.nn.Parameter(t.clone()) for t in case["muon_params"]]
    mu = Muon(lr=hyper["muon_lr"], momentum=hyper["momentum"], weight_decay=hyper["muon_wd"], momentum_dtype=torch.float32)
    for p in pm:
        mu.add_param(p)
    for i, grads in enumerate(case["muon_grads"]):
        for p, g in zip(pm, grads):
            p.grad = g.clone()
        mu.step()
        for p, want, start in zip(pm, ref["muon"][i], case["muon_params"]):
            # the reference runs Newton-Schulz in fp16 (here: fp32 on the CPU), so the orthogonalised update agrees to
            # fp16 rounding through five cubic iterations, not to the last bit
            d_ref, d_here = want - start, p.detach() - start
            cos = torch.nn.functional.cosine_similarity(d_ref.reshape(1, -1), d_here.reshape(1, -1)).item()
            assert cos > 0.999, (i, tuple(p.shape), cos)
            assert abs(d_here.norm().item() / d_ref.norm().item() - 1) < 2e-2, (i, tuple(p.shape))
