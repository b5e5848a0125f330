"""Learning-rate and batch-size schedules (train.py:831-862 of the reference)."""
from __future__ import annotations

import math


def get_lr(base_lr: float, step: int, warmup_steps: int, max_steps: int, cooldown_steps: int = 0,
           schedule: str = "cosine", min_lr: float = 0.0) -> float:
    """Linear warm-up, then cosine | linear | constant/trapezoid, then a linear cool-down that never goes
    below ``min_lr``.  ``step`` counts micro-batch steps, as in the reference."""
    if warmup_steps and step < warmup_steps:
        return base_lr * step / warmup_steps
    if cooldown_steps and step > max_steps - cooldown_steps:
        return max(base_lr * (max_steps - step) / cooldown_steps, min_lr)
    if schedule == "linear":
        return base_lr - (base_lr - min_lr) * (step - warmup_steps) / max(max_steps - warmup_steps, 1)
    if schedule in ("constant", "trapezoid"):
        return base_lr
    if schedule == "cosine":
        frac = (step - warmup_steps) / max(max_steps - warmup_steps, 1)
        return min_lr + (base_lr - min_lr) * (1 + math.cos(math.pi * min(max(frac, 0.0), 1.0))) / 2
    raise ValueError(f"Unsupported lr_schedule: {schedule}")


def get_batch_size(step: int, batch_size_ramp: int, final_accumulation: int) -> int:
    """Gradient-accumulation steps during a linear batch-size ramp (train.py:856-862)."""
    if batch_size_ramp and step < batch_size_ramp:
        return max(math.ceil(step / batch_size_ramp * final_accumulation), 1)
    return final_accumulation
