"""Learning-rate schedules with linear warm-up ``(step+1)/warmup``: cosine, linear, constant, wsd
(constant, then ``1 - sqrt`` decay over the last 20 %). Same curves as the reference's
llmc/schedulers.h:19-98; arithmetic is done in float32 like there. ``get`` evaluates the schedule in the C++ host
library (``llmk_lr_get``); ``get_python`` is the same arithmetic in numpy float32, kept as the cross-check."""
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
        try:
            from . import hostlib
            self._native = hostlib.lib().llmk_lr_get
        except Exception:   # no compiler / library on this machine: numpy path
            self._native = None

    def _warm(self, step: int):
        return self.lr * f32(step + 1) / f32(self.warmup)

    def get(self, step: int) -> float:
        if self._native is None:
            return self.get_python(step)
        v = float(self._native(self.TYPES.index(self.kind), float(self.lr), self.warmup, self.total, float(self.final_frac), int(step)))
        if v != v:
            raise ValueError("step beyond the schedule")
        return v

    def get_python(self, step: int) -> float:
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
