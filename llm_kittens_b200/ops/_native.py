"""ctypes bridge to the in-tree CUDA library (``_lib/libllmk_cuda.so``).

Every op wrapper in this package goes through :func:`call`, which passes raw device pointers and the
current CUDA stream, and turns a non-zero return code into a Python exception. There is no eager
PyTorch fallback behind these wrappers: if the library is missing or fails to load, the ops raise.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Any

import torch

from .. import build as _build

_LOCK = threading.Lock()
_LIB: ctypes.CDLL | None = None

ERRORS = {
    -1: "CUDA runtime error",
    -2: "unsupported or misaligned shape",
    -3: "tensor-map encoding failed",
    -4: "workspace too small",
    -5: "driver entry point missing",
    -6: "size beyond a compiled-in maximum",
}

STATUS_CODES = {
    1: "timeout waiting for a filled TMA stage",
    2: "timeout waiting for a released TMA stage",
    3: "timeout waiting for a finished accumulator",
    4: "timeout waiting for a drained accumulator",
    5: "timeout waiting for a peer flag",
    6: "device-side bounds check failed",
}


class NativeError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load (building first when the shared object is absent) the CUDA library."""
    global _LIB
    if _LIB is None:
        with _LOCK:
            if _LIB is None:
                path = _build.cuda_lib_path()
                if not path.exists():
                    if os.environ.get("LLMK_NO_AUTOBUILD"):
                        raise NativeError(f"{path} is missing; run `python -m llm_kittens_b200.build`")
                    _build.build()
                handle = ctypes.CDLL(str(path))
                handle.llmk_last_error.restype = ctypes.c_char_p
                for fn in ("llmk_gemm_workspace_bytes", "llmk_norm_bwd_scratch_bytes", "llmk_dbias_scratch_bytes",
                           "llmk_bucket_sort_scratch_ints"):
                    getattr(handle, fn).restype = ctypes.c_long
                handle.llmk_optim_grid_x.argtypes = [ctypes.c_long]
                _LIB = handle
    return _LIB


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream_handle() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _conv(a: Any):
    if isinstance(a, torch.Tensor):
        return ctypes.c_void_p(a.data_ptr())
    if a is None:
        return ctypes.c_void_p(0)
    if isinstance(a, bool):
        return ctypes.c_long(int(a))
    if isinstance(a, int):
        # 64-bit slot: correct for both `int` and `long` C parameters on x86-64 / aarch64
        return ctypes.c_long(a)
    if isinstance(a, float):
        return ctypes.c_float(a)
    return a


# kernels launched by one call of a library entry point (default 1); used for the launch counter
_KERNELS_PER_CALL = {"llmk_layernorm_bwd": 2, "llmk_rmsnorm_bwd": 2, "llmk_dbias": 2, "llmk_attention_bwd": 3, "llmk_attention_bwd_tc": 2,
                     "llmk_encoder_bwd": 2, "llmk_global_norm2": 2, "llmk_bucket_sort": 6, "llmk_moe_dispatch_signal": 2, "llmk_moe_dispatch": 2,
                     "llmk_dbias_grouped": 2, "llmk_attention_bwd_tc_rope": 2, "llmk_attention_bwd_ring_step": 2}
_LAUNCHES = 0


def launch_count() -> int:
    """Number of kernels of this library launched so far by this process (split-K GEMMs count their
    reduction kernel as well)."""
    return _LAUNCHES


def count_replayed(kernels: int) -> None:
    """A captured CUDA graph with ``kernels`` of this library's kernels has been replayed once."""
    global _LAUNCHES
    _LAUNCHES += kernels


# ---- step ledger: device time of every library call inside a running step ------------------------------------
_LEDGER: list | None = None


def ledger_start() -> None:
    """From now on every :func:`call` is bracketed by two CUDA events on its stream (no synchronisation)."""
    global _LEDGER
    _LEDGER = []


def ledger_stop() -> dict[str, tuple[int, float]]:
    """Synchronise and return {label: (calls, total milliseconds)}. GEMM calls are labelled by layout, epilogue and
    shape, other entry points by name."""
    global _LEDGER
    rows, _LEDGER = _LEDGER or [], None
    torch.cuda.synchronize()
    out: dict[str, tuple[int, float]] = {}
    for label, e0, e1 in rows:
        n, ms = out.get(label, (0, 0.0))
        out[label] = (n + 1, ms + e0.elapsed_time(e1))
    return out


def _ledger_label(name: str, args) -> str:
    if name in ("llmk_gemm", "llmk_gemm_grouped"):
        mode, epi = args[0], args[1]
        M, Nn, K = args[8], args[9], args[10]
        return f"{name[5:]} {('NT', 'NN', 'TN')[mode]} epi={epi} {M}x{Nn}x{K}"
    if name == "llmk_gemm_tn_dbias":
        return f"gemm TN +dbias {args[5]}x{args[6]}x{args[7]}"
    return name[5:]


def call(name: str, *args: Any) -> None:
    """Call ``int name(args..., void* stream)``; tensors become device pointers; raises on failure."""
    global _LAUNCHES
    fn = getattr(lib(), name)
    if _LEDGER is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = fn(*[_conv(a) for a in args], stream_handle())
        e1.record()
        _LEDGER.append((_ledger_label(name, args), e0, e1))
    else:
        rc = fn(*[_conv(a) for a in args], stream_handle())
    _LAUNCHES += _KERNELS_PER_CALL.get(name, 1)
    if rc != 0:
        detail = lib().llmk_last_error().decode() if rc == -1 else ""
        raise NativeError(f"{name} failed: {ERRORS.get(rc, rc)} {detail}")


_STATUS: dict[int, torch.Tensor] = {}


def status_word() -> torch.Tensor:
    """Per-device int32[4] that kernels with bounded waits write their failure code into."""
    dev = torch.cuda.current_device()
    if dev not in _STATUS:
        _STATUS[dev] = torch.zeros(4, dtype=torch.int32, device=f"cuda:{dev}")
        with torch.cuda.device(dev):
            lib().llmk_set_status_word(ctypes.c_void_p(_STATUS[dev].data_ptr()))
    return _STATUS[dev]


def check_status(reset: bool = True) -> None:
    """Synchronise and raise if any kernel recorded a bounded-wait failure since the last check."""
    st = status_word()
    vals = st.tolist()
    if vals[0] != 0:
        if reset:
            st.zero_()
        raise NativeError(
            f"kernel reported status {vals[0]} ({STATUS_CODES.get(vals[0], '?')}), tag={vals[1]} block={vals[2]} thread={vals[3]}"
        )


def require_cuda_tensor(t: torch.Tensor, dtype: torch.dtype | None = None, name: str = "tensor") -> None:
    if not t.is_cuda:
        raise NativeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise NativeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise NativeError(f"{name} must be {dtype}, got {t.dtype}")


# ---- guard regions around scratch buffers ---------------------------------------------------------------
# compute-sanitizer is not available where this runs, so the scratch buffers that kernels write through raw
# pointers (split-K partials, column-sum partials of the norm / bias gradients) can be allocated with a canary
# page on each side; check_guards() verifies them on the host. Off by default (the buffers are then pooled and
# oversized); LLMK_GUARD=1 or set_guards(True) turns it on, which the GPU tests do.
_GUARD_BYTES = 4096
_GUARD_VALUE = 0xA5
_GUARDS_ON = os.environ.get("LLMK_GUARD", "0") not in ("", "0")
_GUARDED: list[tuple[str, torch.Tensor, int]] = []   # (name, whole allocation, payload bytes)


def set_guards(on: bool) -> None:
    global _GUARDS_ON
    _GUARDS_ON = bool(on)
    if not on:
        _GUARDED.clear()


def guards_enabled() -> bool:
    return _GUARDS_ON


def scratch_buffer(pool: dict, nbytes: int, min_bytes: int, name: str) -> torch.Tensor:
    """A uint8 device buffer of at least ``nbytes`` from ``pool`` (one per device). With guards on it is exactly
    ``nbytes`` (rounded up to 256) between two canary regions, so that a kernel writing past its stated need is seen."""
    dev = torch.cuda.current_device()
    if not _GUARDS_ON:
        s = pool.get(dev)
        if s is None or s.numel() < nbytes:
            s = torch.empty(max(nbytes, min_bytes), dtype=torch.uint8, device=f"cuda:{dev}")
            pool[dev] = s
        return s
    payload = (max(nbytes, 1) + 255) // 256 * 256
    key = (dev, "guarded", payload)
    whole = pool.get(key)
    if whole is None:
        whole = torch.full((payload + 2 * _GUARD_BYTES,), _GUARD_VALUE, dtype=torch.uint8, device=f"cuda:{dev}")
        pool[key] = whole
        _GUARDED.append((f"{name}[{payload}]@cuda:{dev}", whole, payload))
    return whole[_GUARD_BYTES:_GUARD_BYTES + payload]


def check_guards() -> int:
    """Synchronise and verify every canary region; returns the number of guarded buffers, raises on damage."""
    for name, whole, payload in _GUARDED:
        lo = whole[:_GUARD_BYTES]
        hi = whole[_GUARD_BYTES + payload:]
        if not bool((lo == _GUARD_VALUE).all().item()) or not bool((hi == _GUARD_VALUE).all().item()):
            raise NativeError(f"guard region of scratch buffer {name} was overwritten")
    return len(_GUARDED)
