"""Learning-rate schedule used by the SciAgent trainers
(scirust-sciagent/src/train/scheduler.rs:3-40): linear warm-up from 0, cosine decay to
``min_lr`` at ``total_steps``, constant ``min_lr`` afterwards. Arithmetic is done in fp32 steps
like the reference so resumed runs reproduce the same values."""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass
class WarmupCosineSchedule:
    base: float
    min_lr: float
    warmup_steps: int
    total_steps: int

    def lr_at(self, step: int) -> float:
        f = np.float32
        if step < self.warmup_steps:
            return float(f(self.base) * (f(step) / f(self.warmup_steps)))
        post = step - self.warmup_steps
        period = self.total_steps - self.warmup_steps
        if post >= period:
            return float(f(self.min_lr))
        progress = f(post) / f(period)
        cos_factor = f(0.5) * (f(1.0) + f(math.cos(float(f(math.pi) * progress))))
        return float(f(self.min_lr) + (f(self.base) - f(self.min_lr)) * cos_factor)


@dataclass
class ConstantSchedule:
    base: float

    def lr_at(self, step: int) -> float:
        return self.base
