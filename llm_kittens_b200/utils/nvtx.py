"""NVTX ranges for the trainer phases and op groups.

The reference opens an ``NvtxRange`` at the top of every op wrapper and trainer phase (llmc/cuda_common.h:87-96,
train_gpt2.cu:801, 839, 929, 2111, 2117) and brackets the first steps with cudaProfilerStart / cudaProfilerStop
(train_gpt2.cu:2105-2107, 2319-2323). Here the ranges go through ``torch.cuda.nvtx``; they are off unless
``LLMK_NVTX=1`` (a push / pop pair costs a few microseconds of host time per range, which a launch-bound step
would notice), and the recorded names are kept in a small ring so that CPU tests can check the nesting.
"""
from __future__ import annotations

import contextlib
import os

import torch

_ENABLED = os.environ.get("LLMK_NVTX", "0") not in ("", "0")
_TRACE: list[tuple[str, int]] = []   # (name, depth) of the most recent ranges, newest last
_DEPTH = 0
_TRACE_MAX = 256


def enabled() -> bool:
    return _ENABLED


def set_enabled(on: bool) -> None:
    global _ENABLED
    _ENABLED = bool(on)


def recent() -> list[tuple[str, int]]:
    """(name, nesting depth) of the ranges opened most recently (at most 256)."""
    return list(_TRACE)


@contextlib.contextmanager
def nvtx_range(name: str):
    """``with nvtx_range("forward"):`` — a named range on the calling thread; a no-op when disabled."""
    global _DEPTH
    if not _ENABLED:
        yield
        return
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.nvtx.range_push(name)
    _TRACE.append((name, _DEPTH))
    if len(_TRACE) > _TRACE_MAX:
        del _TRACE[0]
    _DEPTH += 1
    try:
        yield
    finally:
        _DEPTH -= 1
        if cuda:
            torch.cuda.nvtx.range_pop()


def profiler_start() -> None:
    """cudaProfilerStart: lets ``nsys --capture-range=cudaProfilerApi`` / ncu limit the capture to the steps
    between this call and :func:`profiler_stop`."""
    if _ENABLED and torch.cuda.is_available():
        torch.cuda.profiler.start()


def profiler_stop() -> None:
    if _ENABLED and torch.cuda.is_available():
        torch.cuda.profiler.stop()
