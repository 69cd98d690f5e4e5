"""Warmup-stable-decay learning-rate schedule: linear warmup over `warmup_steps`, constant, linear decay over the
last `decay_fraction` of the run to `lr_floor` x peak (reference: ced/train/trainer.py:638-655)."""

from __future__ import annotations


def lr_schedule(optim, total: int, step: int | float) -> float:
    decay_start = int(total * (1.0 - optim.decay_fraction))
    if step < optim.warmup_steps:
        return optim.lr * min(step + 1, optim.warmup_steps) / optim.warmup_steps
    if step < decay_start:
        return optim.lr
    left = max(0.0, (total - step) / max(1, total - decay_start))
    floor = getattr(optim, "lr_floor", 0.0)
    return optim.lr * (floor + (1.0 - floor) * left) if floor else optim.lr * left


def lr_of(cfg, step: int) -> float:
    total = cfg.steps if cfg.optim.schedule_steps is None else cfg.optim.schedule_steps
    return lr_schedule(cfg.optim, total, step)
