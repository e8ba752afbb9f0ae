"""Autoregressive sampling for the periodic "generating:" print-out of the trainers.

Like the reference (train_gpt2.cu:2150-2194) the whole (1, T) window is re-run for every new token
(T rounded up to a multiple of 64 here), the logits of the last real position are copied to the
host, and the next token is drawn from the softmax with the xorshift* coin stream. It is a
diagnostic path, not a serving engine.
"""
from __future__ import annotations

import numpy as np
import torch

from ..utils.rand import Xorshift, sample_softmax


@torch.no_grad()
def generate(model, prompt: list[int], num_tokens: int, rng_state: int = 1337) -> list[int]:
    cfg = model.config
    rng = Xorshift(rng_state)
    toks = list(prompt)
    # The model is re-run on (1, T) windows, which makes it reallocate everything that depends on the shape: the
    # activations, the token / target buffers and, in a mixture-of-experts model, the routing and exchange buffers with
    # their capacities. All of it is put back afterwards by restoring the model's attribute table, so the training-shape
    # tensors are the very same objects as before (a captured CUDA graph of the micro-step keeps their addresses).
    saved = dict(model.__dict__)
    pad_to = 64
    limit = min(num_tokens, cfg.max_seq_len)
    eot = prompt[0] if prompt else 0
    try:
        while len(toks) < limit:
            t = len(toks)
            T = min(cfg.max_seq_len, ((t + pad_to - 1) // pad_to) * pad_to)
            window = toks + [eot] * (T - t)
            x = torch.tensor([window], dtype=torch.int32, device=model.device)
            if (model.B, model.T) != (1, T):
                model.acts = None
            model.forward(x, None)
            logits = model.logits_view()[0, t - 1, : cfg.vocab_size].float().cpu().numpy()
            toks.append(sample_softmax(np.ascontiguousarray(logits), rng.f32()))
    finally:
        model.__dict__.clear()
        model.__dict__.update(saved)
    return toks
