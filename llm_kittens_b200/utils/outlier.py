"""Rolling z-score over a 128-sample window (double precision); NaN until the window is full.
Used for the ``-sl`` / ``-sg`` skip-update guards (reference llmc/outlier_detector.h:16-70)."""
from __future__ import annotations

import math

WINDOW = 128


class OutlierDetector:
    def __init__(self):
        self.buffer = [0.0] * WINDOW
        self.count = 0
        self.index = 0
        self.sum = 0.0
        self.sum_sq = 0.0

    def update(self, value: float) -> float:
        value = float(value)
        if self.count < WINDOW:
            self.buffer[self.count] = value
            self.sum += value
            self.sum_sq += value * value
            self.count += 1
            return float("nan")
        old = self.buffer[self.index]
        self.sum += value - old
        self.sum_sq += value * value - old * old
        self.buffer[self.index] = value
        self.index = (self.index + 1) % WINDOW
        mean = self.sum / WINDOW
        var = self.sum_sq / WINDOW - mean * mean
        std = math.sqrt(var) if var > 0 else 0.0
        if std == 0.0:
            return 0.0
        return (value - mean) / std


class NativeOutlierDetector:
    """The same detector inside the C++ host library (``llmk_outlier_*``)."""

    def __init__(self):
        from . import hostlib

        self._lib = hostlib.lib()
        self._h = self._lib.llmk_outlier_create()

    def update(self, value: float) -> float:
        return float(self._lib.llmk_outlier_update(self._h, float(value)))

    def __del__(self):
        try:
            self._lib.llmk_outlier_destroy(self._h)
        except Exception:
            pass
