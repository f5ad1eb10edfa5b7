"""Learning-rate schedules (scirust-core/src/autodiff/scheduler.rs:39-305): ``lr_at(step)`` is a
pure function of the step, except ``ReduceOnPlateau`` which reacts to a monitored metric."""
from __future__ import annotations

import math


class LrSchedule:
    def lr_at(self, step: int) -> float:
        raise NotImplementedError

    def apply(self, optimizer, step: int) -> float:
        lr = self.lr_at(step)
        optimizer.set_lr(lr)
        return lr


class Constant(LrSchedule):
    def __init__(self, lr: float):
        self.lr = lr

    def lr_at(self, step):
        return self.lr


class StepDecay(LrSchedule):
    def __init__(self, base: float, step_size: int, gamma: float):
        self.base, self.step_size, self.gamma = base, max(1, step_size), gamma

    def lr_at(self, step):
        return self.base * self.gamma ** (step // self.step_size)


class Exponential(LrSchedule):
    def __init__(self, base: float, gamma: float):
        self.base, self.gamma = base, gamma

    def lr_at(self, step):
        return self.base * self.gamma ** step


class CosineAnnealing(LrSchedule):
    def __init__(self, base: float, min_lr: float, t_max: int):
        self.base, self.min_lr, self.t_max = base, min_lr, max(1, t_max)

    def lr_at(self, step):
        t = min(step, self.t_max)
        return self.min_lr + 0.5 * (self.base - self.min_lr) * (1.0 + math.cos(math.pi * t / self.t_max))


class WarmupCosine(LrSchedule):
    def __init__(self, base: float, min_lr: float, warmup_steps: int, total_steps: int):
        self.base, self.min_lr, self.warmup_steps, self.total_steps = base, min_lr, warmup_steps, total_steps

    def lr_at(self, step):
        if step < self.warmup_steps:
            return self.base * step / max(1, self.warmup_steps)
        period = max(1, self.total_steps - self.warmup_steps)
        post = step - self.warmup_steps
        if post >= period:
            return self.min_lr
        return self.min_lr + 0.5 * (self.base - self.min_lr) * (1.0 + math.cos(math.pi * post / period))


class ReduceOnPlateau(LrSchedule):
    """Multiply the rate by ``factor`` after ``patience`` evaluations without improvement."""

    def __init__(self, base: float, factor: float = 0.1, patience: int = 10, min_lr: float = 0.0,
                 threshold: float = 1e-4):
        self.lr, self.factor, self.patience, self.min_lr, self.threshold = base, factor, patience, min_lr, threshold
        self.best, self.bad = float("inf"), 0

    def observe(self, metric: float) -> float:
        if metric < self.best - self.threshold:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
            if self.bad > self.patience:
                self.lr = max(self.min_lr, self.lr * self.factor)
                self.bad = 0
        return self.lr

    def lr_at(self, step):
        return self.lr
