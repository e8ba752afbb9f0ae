"""Random numbers: an MT19937 generator whose ``normal_`` / ``uniform_`` / permutation streams equal
``torch.manual_seed`` + CPU ``torch.normal`` (so initial weights can be reproduced bit for bit, as the
reference does with llmc/rand.h), and the xorshift* stream that seeds stochastic rounding."""
from __future__ import annotations

import ctypes

import numpy as np

from . import hostlib


class Mt19937:
    def __init__(self, seed: int = 5489):
        self._h = hostlib.lib().llmk_rng_create(seed & 0xFFFFFFFF)

    def __del__(self):
        try:
            hostlib.lib().llmk_rng_destroy(self._h)
        except Exception:
            pass

    def seed(self, seed: int) -> None:
        hostlib.lib().llmk_rng_seed(self._h, seed & 0xFFFFFFFF)

    def randint32(self) -> int:
        return int(hostlib.lib().llmk_rng_u32(self._h))

    def normal_(self, n: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        hostlib.lib().llmk_rng_normal(self._h, out.ctypes.data, n, mean, std)
        return out

    def uniform_(self, n: int, lo: float = 0.0, hi: float = 1.0) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        hostlib.lib().llmk_rng_uniform(self._h, out.ctypes.data, n, lo, hi)
        return out

    def permutation(self, n: int) -> np.ndarray:
        data = np.arange(n, dtype=np.int32)
        hostlib.lib().llmk_rng_permutation(self._h, data.ctypes.data, n)
        return data

    def state(self) -> bytes:
        buf = ctypes.create_string_buffer(hostlib.lib().llmk_rng_state_bytes())
        hostlib.lib().llmk_rng_save(self._h, buf)
        return buf.raw

    def set_state(self, blob: bytes) -> None:
        hostlib.lib().llmk_rng_load(self._h, ctypes.create_string_buffer(blob, len(blob)))


class Xorshift:
    """64-bit xorshift* state; ``u32()`` gives the per-step / per-tensor seeds for stochastic rounding."""

    def __init__(self, state: int = 13371337):
        self._s = ctypes.c_uint64(state)

    @property
    def state(self) -> int:
        return int(self._s.value)

    @state.setter
    def state(self, v: int) -> None:
        self._s.value = v

    def u32(self) -> int:
        return int(hostlib.lib().llmk_xorshift_u32(ctypes.byref(self._s)))

    def f32(self) -> float:
        return float(hostlib.lib().llmk_xorshift_f32(ctypes.byref(self._s)))


def sample_softmax(logits: np.ndarray, coin: float) -> int:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    return int(hostlib.lib().llmk_sample_softmax(logits.ctypes.data, logits.size, coin))
