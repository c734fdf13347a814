"""First-steps diagnostics on small real optimizers: max-abs scans and non-finite counts."""
import logging

import torch
import torch.nn as nn


def _opts():
    from hippolm_b200.optim.optimizers import Muon, AdamW
    w = nn.Parameter(torch.full((8, 16), 0.5))
    b = nn.Parameter(torch.full((16,), -2.0))
    w.grad = torch.full_like(w, 3.0)
    b.grad = torch.full_like(b, -0.25)
    muon = Muon(lr=0.02, momentum_dtype=torch.float32); muon.add_param(w, "w")
    adamw = AdamW(lr=0.004, m_dtype=torch.float32, v_dtype=torch.float32); adamw.add_param(b, "b")
    return muon, adamw, w, b


def test_optimizer_stats_and_pre_step_log():
    from hippolm_b200.train.diagnostics import optimizer_stats, log_pre_step_diag
    muon, adamw, w, b = _opts()
    s = optimizer_stats(muon)
    assert s["grad_max"] == 3.0 and s["param_max"] == 0.5 and s["exp_avg_max"] == 0.0
    s = optimizer_stats(adamw)
    assert s["grad_max"] == 0.25 and s["param_max"] == 2.0 and s["exp_avg_sq_max"] == 0.0
    out = log_pre_step_diag(logging.getLogger("diag-test"), 0, [muon, adamw], 1.5)
    assert out["grad_norm"] == 1.5 and out["Muon"]["grad_max"] == 3.0 and out["AdamW"]["param_max"] == 2.0


def test_non_finite_scan_after_a_step():
    from hippolm_b200.train.diagnostics import count_non_finite, log_post_opt_diag
    muon, adamw, w, b = _opts()
    muon.step(); adamw.step()
    assert count_non_finite(muon) == 0 and count_non_finite(adamw) == 0
    adamw.entries[0].exp_avg[3] = float("nan")
    w.data[0, 0] = float("inf")
    out = log_post_opt_diag(logging.getLogger("diag-test"), 1, [muon, adamw])
    assert out["Muon_non_finite"] == 1 and out["AdamW_non_finite"] == 1
