"""Warmup-stable-decay learning-rate schedule (``src/training/loop/support.py:29-89``)."""
from __future__ import annotations


def wsd_lr(step: int, peak_lr: float, warmup_steps: int, decay_steps: int, max_steps: int,
           min_lr: float = 0.0) -> float:
    """lr(step): linear warmup ``peak*step/warmup``; constant ``peak``; linear decay to ``min_lr``
    over the last ``decay_steps`` steps with divisor ``decay_steps - 1`` (so the final step lands on
    ``min_lr`` exactly); 0 outside ``[0, max_steps)``."""
    if peak_lr <= 0.0:
        return peak_lr
    if step < 0 or step >= max_steps:
        return 0.0
    if warmup_steps > 0 and step < warmup_steps:
        return peak_lr * step / warmup_steps
    decay_start = max_steps - decay_steps
    if decay_steps > 0 and step >= decay_start:
        frac = (step - decay_start) / (decay_steps - 1 if decay_steps > 1 else 1)
        return peak_lr + (min_lr - peak_lr) * frac
    return peak_lr
