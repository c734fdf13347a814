"""CUDA path of the optimizer update kernels."""
from __future__ import annotations

import torch


def adamw_update(p, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    gf = g.float() * grad_scale
    mf = m.float().mul_(beta1).add_(gf, alpha=1 - beta1)
    vf = v.float().mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    m.copy_(mf); v.copy_(vf)
    upd = (mf / (1 - beta1 ** step)) / ((vf / (1 - beta2 ** step)).sqrt() + eps)
    p.copy_(p.float().mul_(1 - lr * wd).add_(upd, alpha=-lr))
