"""Python faces of the C++ loaders (``csrc/host/llmk_host.cpp``).

:class:`DataLoader` streams ``(B, T)`` input / target batches out of token shards: rank ``r`` of ``P``
reads the ``r``-th ``B*T`` slice of every global batch of ``P*B*T`` tokens, optionally in shuffled
shard / sample order (reference llmc/dataloader.h:27-323). Batches are written straight into pinned
int32 tensors so the trainer can issue one asynchronous host-to-device copy per micro-step.
:class:`EvalLoader` packs multiple-choice examples four rows at a time (llmc/dataloader.h:344-660).
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import hostlib


def _pinned(shape, dtype):
    try:
        return torch.empty(shape, dtype=dtype, pin_memory=torch.cuda.is_available())
    except RuntimeError:
        return torch.empty(shape, dtype=dtype)


class DataLoader:
    def __init__(self, pattern: str, B: int, T: int, process_rank: int = 0, num_processes: int = 1, should_shuffle: bool = False,
                 ring: int = 2):
        """``ring``: number of pinned batch buffers that are cycled through. A batch handed out stays
        untouched for the next ``ring - 1`` calls. Its consumer copies it to the device asynchronously, so
        before a buffer is refilled the loader waits for a CUDA event that it recorded (on the stream current
        at that time) when the consumer came back for the following batch, i.e. after that copy had been
        queued: a loop that queues work faster than the GPU runs it is held back to ``ring - 1`` batches
        ahead instead of overwriting tokens that have not been copied yet."""
        self.B, self.T = B, T
        self._lib = hostlib.lib()
        self._h = self._lib.llmk_loader_create(pattern.encode(), B, T, process_rank, num_processes, int(should_shuffle))
        if not self._h:
            raise hostlib.HostError(hostlib.last_error())
        self.should_shuffle = should_shuffle
        self._ring = [(_pinned((B, T), torch.int32), _pinned((B, T), torch.int32)) for _ in range(max(1, ring))]
        self._slot = 0
        self._events = [None] * len(self._ring)
        self._cuda = torch.cuda.is_available() and self._ring[0][0].is_pinned()
        self.inputs, self.targets = self._ring[0]
        self.num_tokens = int(self._lib.llmk_loader_num_tokens(self._h))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.llmk_loader_destroy(self._h)
            self._h = None

    __del__ = close

    def next_batch(self):
        """Advance to the next batch; returns the (pinned, recycled) ``inputs`` and ``targets`` tensors."""
        if self._cuda:
            # everything queued so far includes the upload of the batch handed out last
            ev = self._events[self._slot] or torch.cuda.Event()
            ev.record()
            self._events[self._slot] = ev
        self._slot = (self._slot + 1) % len(self._ring)
        if self._events[self._slot] is not None:
            self._events[self._slot].synchronize()
        self.inputs, self.targets = self._ring[self._slot]
        if self._lib.llmk_loader_next(self._h, self.inputs.data_ptr(), self.targets.data_ptr()) != 0:
            raise hostlib.HostError(hostlib.last_error())
        return self.inputs, self.targets

    def reset(self):
        if self._lib.llmk_loader_reset(self._h) != 0:
            raise hostlib.HostError(hostlib.last_error())

    def resume(self, shard_idx: int, sample_idx: int, shuffle_blob: bytes = b""):
        if self.should_shuffle and shuffle_blob:
            buf = ctypes.create_string_buffer(shuffle_blob, len(shuffle_blob))
            if self._lib.llmk_loader_load_shuffle_state(self._h, buf, len(shuffle_blob)) != 0:
                raise hostlib.HostError(hostlib.last_error())
        if self._lib.llmk_loader_resume(self._h, shard_idx, sample_idx) != 0:
            raise hostlib.HostError(hostlib.last_error())

    @property
    def current_shard_idx(self) -> int:
        return int(self._lib.llmk_loader_shard_idx(self._h))

    @property
    def current_sample_idx(self) -> int:
        return int(self._lib.llmk_loader_sample_idx(self._h))

    @property
    def num_shards(self) -> int:
        return int(self._lib.llmk_loader_num_shards(self._h))

    def shuffle_state(self) -> bytes:
        n = int(self._lib.llmk_loader_shuffle_state_bytes(self._h))
        if n == 0:
            return b""
        buf = ctypes.create_string_buffer(n)
        self._lib.llmk_loader_save_shuffle_state(self._h, buf)
        return buf.raw


class EvalLoader:
    NUM_COMPLETIONS = 4

    def __init__(self, path: str, B: int, T: int, process_rank: int = 0, num_processes: int = 1):
        self.B, self.T = B, T
        self._lib = hostlib.lib()
        self._h = self._lib.llmk_evalloader_create(path.encode(), B, T, process_rank, num_processes)
        if not self._h:
            raise hostlib.HostError(hostlib.last_error())
        self.inputs = _pinned((B, T), torch.int32).zero_()
        self.targets = _pinned((B, T), torch.int32).zero_()
        self.mask = torch.zeros(B, T, dtype=torch.int8)
        self.label = torch.zeros(max(1, B // 4), dtype=torch.int32)
        self.num_examples = int(self._lib.llmk_evalloader_num_examples(self._h))
        self.num_batches = int(self._lib.llmk_evalloader_num_batches(self._h))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.llmk_evalloader_destroy(self._h)
            self._h = None

    __del__ = close

    def reset(self):
        if self._lib.llmk_evalloader_reset(self._h) != 0:
            raise hostlib.HostError(hostlib.last_error())

    def next_batch(self):
        rc = self._lib.llmk_evalloader_next(self._h, self.inputs.data_ptr(), self.targets.data_ptr(), self.mask.data_ptr(),
                                            self.label.data_ptr())
        if rc != 0:
            raise hostlib.HostError(hostlib.last_error())
        return self.inputs, self.targets

    def stat_losses(self, losses) -> int:
        """Number of examples in the current batch whose lowest mean masked loss is the labelled completion."""
        arr = np.ascontiguousarray(np.asarray(losses, dtype=np.float32).reshape(self.B, self.T))
        return int(self._lib.llmk_evalloader_stat_losses(arr.ctypes.data, self.mask.data_ptr(), self.label.data_ptr(), self.B, self.T))
