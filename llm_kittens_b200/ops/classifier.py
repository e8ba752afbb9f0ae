"""Fused softmax + cross-entropy (+ in-place dlogits) (``csrc/classifier.cu``); reference job:
fused_classifier (llmc/fused_classifier.cuh:240-258)."""
from __future__ import annotations

import torch

from . import _native as N


def fused_classifier(logits, targets, V, dloss, losses=None, write_dlogits=True, accumulate_loss=False):
    """``logits``: [rows, Vp] bf16 (overwritten by dlogits when ``write_dlogits``); returns per-row losses."""
    rows, Vp = logits.shape
    losses = torch.empty(rows, dtype=torch.float32, device=logits.device) if losses is None else losses
    N.call("llmk_fused_classifier", logits, losses, targets, float(dloss), rows, V, Vp, int(write_dlogits), int(accumulate_loss))
    return losses


def sum_scaled(out, x, scale, accumulate=False):
    """``out[0] (+)= scale * sum(x)`` with a fixed summation order."""
    N.call("llmk_sum_scaled", out, x, x.numel(), float(scale), int(accumulate))
    return out
