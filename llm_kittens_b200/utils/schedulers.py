"""Learning-rate schedules with linear warm-up ``(step+1)/warmup``: cosine, linear, constant, wsd
(constant, then ``1 - sqrt`` decay over the last 20 %). Same curves as the reference's
llmc/schedulers.h:19-98; arithmetic is done in float32 like there."""
from __future__ import annotations

import math

import numpy as np

f32 = np.float32


class LearningRateScheduler:
    TYPES = ("cosine", "linear", "constant", "wsd")

    def __init__(self, kind: str, learning_rate: float, warmup_iterations: int, train_num_batches: int,
                 final_learning_rate_frac: float):
        if kind not in self.TYPES:
            raise ValueError(f"Unknown learning rate scheduler type: {kind}")
        self.kind = kind
        self.lr = f32(learning_rate)
        self.warmup = int(warmup_iterations)
        self.total = int(train_num_batches)
        self.final_frac = f32(final_learning_rate_frac)

    def _warm(self, step: int):
        return self.lr * f32(step + 1) / f32(self.warmup)

    def get(self, step: int) -> float:
        lr, min_lr = self.lr, self.lr * self.final_frac
        if self.kind == "constant":
            return float(lr)
        if step < self.warmup:
            return float(self._warm(step))
        if self.kind == "wsd":
            decay_point = int(f32(0.8) * f32(self.total))
            if step < decay_point:
                return float(lr)
            ratio = f32(step - decay_point) / f32(self.total - decay_point)
            return float(min_lr + (f32(1.0) - f32(math.sqrt(ratio))) * (lr - min_lr))
        ratio = f32(step - self.warmup) / f32(self.total - self.warmup)
        if not (0.0 <= ratio <= 1.0):
            raise ValueError("step beyond the schedule")
        if self.kind == "cosine":
            coeff = f32(0.5) * (f32(1.0) + f32(math.cos(math.pi * float(ratio))))
            return float(min_lr + coeff * (lr - min_lr))
        return float(lr - ratio * (lr - min_lr))
