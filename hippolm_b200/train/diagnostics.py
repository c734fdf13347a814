"""First-steps diagnostics: max-abs of gradients / moments / parameters and finite scans
(``src/training/diagnostics.py:36-176``)."""
from __future__ import annotations

from typing import Dict, List

import torch


def _max_abs(ts) -> float:
    m = 0.0
    for t in ts:
        if t is not None and t.numel():
            m = max(m, float(t.detach().float().abs().max()))
    return m


def optimizer_stats(opt) -> Dict[str, float]:
    grads = [e.grad() for e in opt.entries]
    params = [e.param.data for e in opt.entries if e.param is not None]
    return {"grad_max": _max_abs(grads), "exp_avg_max": _max_abs([e.exp_avg for e in opt.entries]),
            "exp_avg_sq_max": _max_abs([e.exp_avg_sq for e in opt.entries if e.exp_avg_sq is not None]),
            "param_max": _max_abs(params)}


def count_non_finite(opt) -> int:
    n = 0
    for e in opt.entries:
        for t in (e.param.data if e.param is not None else None, e.exp_avg, e.exp_avg_sq):
            if t is not None:
                n += int((~torch.isfinite(t.float())).sum())
    return n


def log_pre_step_diag(logger, step: int, opts: List, grad_norm: float) -> Dict:
    out = {"step": step, "grad_norm": grad_norm}
    for o in opts:
        out[type(o).__name__] = optimizer_stats(o)
    logger.info(f"[diag pre] {out}")
    return out


def log_post_opt_diag(logger, step: int, opts: List) -> Dict:
    out = {"step": step}
    for o in opts:
        out[type(o).__name__ + "_non_finite"] = count_non_finite(o)
    logger.info(f"[diag post] {out}")
    return out
