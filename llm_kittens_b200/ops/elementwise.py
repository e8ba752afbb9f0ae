"""Element-wise kernels (``csrc/elementwise.cu``): GELU, SwiGLU, RoPE, adds, bias gradient, encoder.
Reference jobs: llmc/gelu.cuh, llmc/swiglu.cuh, llmc/rope.cuh, llmc/encoder.cuh, matmul_backward_bias."""
from __future__ import annotations

import torch

from . import _native as N

_DBIAS_SCRATCH: dict[int, torch.Tensor] = {}


def gelu_fwd(inp, out=None):
    out = torch.empty_like(inp) if out is None else out
    N.call("llmk_gelu_fwd", out, inp, inp.numel())
    return out


def gelu_bwd_inplace(dinout, inp):
    N.call("llmk_gelu_bwd_inplace", dinout, inp, inp.numel())
    return dinout


def swiglu_fwd(gate, up, out=None):
    out = torch.empty_like(gate) if out is None else out
    N.call("llmk_swiglu_fwd", out, gate, up, gate.numel())
    return out


def swiglu_bwd(dout, gate, up, dgate=None, dup=None):
    dgate = torch.empty_like(gate) if dgate is None else dgate
    dup = torch.empty_like(up) if dup is None else dup
    N.call("llmk_swiglu_bwd", dgate, dup, dout, gate, up, gate.numel())
    return dgate, dup


def swiglu_fused_fwd(upgate, out=None):
    """``upgate``: [rows, 2H] with up in the first H columns and gate in the last H."""
    rows, H2 = upgate.shape
    H = H2 // 2
    out = torch.empty(rows, H, dtype=upgate.dtype, device=upgate.device) if out is None else out
    N.call("llmk_swiglu_fused_fwd", out, upgate, rows, H)
    return out


def swiglu_fused_bwd(dout, upgate, dupgate=None):
    rows, H2 = upgate.shape
    dupgate = torch.empty_like(upgate) if dupgate is None else dupgate
    N.call("llmk_swiglu_fused_bwd", dupgate, dout, upgate, rows, H2 // 2)
    return dupgate


def add(a, b, out=None):
    out = torch.empty_like(a) if out is None else out
    N.call("llmk_add", out, a, b, a.numel())
    return out


def rope_tables(T: int, HS: int, theta: float = 500000.0, scaled: bool = False, device="cuda") -> torch.Tensor:
    """[T, HS/2, 2] fp32 (cos, sin); optional Llama-3.1 frequency scaling (factor 8, low 1, high 4,
    original context 8192) as in the reference's table builder (train_llama3.cu:303-347)."""
    import math

    inv = 1.0 / (theta ** (torch.arange(0, HS, 2, dtype=torch.float64) / HS))
    if scaled:
        factor, low, high, old = 8.0, 1.0, 4.0, 8192.0
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - low) / (high - low)
        scaled_inv = torch.where(wavelen < old / high, inv, torch.where(wavelen > old / low, inv / factor,
                                                                        (1 - smooth) * inv / factor + smooth * inv))
        inv = scaled_inv
    ang = torch.outer(torch.arange(T, dtype=torch.float64), inv)
    return torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device).contiguous()


def rope_qk_(qkv, freqs, B, T, NH, NKVH, HS, interleaved=True, inverse=False):
    """Rotate the q and k heads of packed ``qkv`` in place (``inverse`` = backward)."""
    N.call("llmk_rope_qk", qkv, freqs, B, T, NH, NKVH, HS, int(interleaved), int(inverse))
    return qkv


def dbias(dbias_t, dout, accumulate=True):
    rows, OC = dout.shape
    nbytes = int(N.lib().llmk_dbias_scratch_bytes(rows, OC))
    # partial sums of its own: the model runs these column sums on a side stream while norm kernels use theirs
    N.call("llmk_dbias", dbias_t, N.scratch_buffer(_DBIAS_SCRATCH, nbytes, 1 << 20, "bias-gradient partials"), dout, rows, OC,
           int(accumulate))
    return dbias_t


def dbias_grouped(dbias_t, dout, groups, accumulate=True):
    """``dbias_t`` [groups, OC] (+)= column sums of each of the ``groups`` equal row blocks stacked in ``dout``."""
    rows, OC = dout.shape[0] // groups, dout.shape[1]
    if groups == 1 or not hasattr(N.lib(), "llmk_dbias_grouped"):
        for g in range(groups):
            dbias(dbias_t[g], dout[g * rows:(g + 1) * rows], accumulate)
        return dbias_t
    nbytes = groups * int(N.lib().llmk_dbias_scratch_bytes(rows, OC))
    N.call("llmk_dbias_grouped", dbias_t, N.scratch_buffer(_DBIAS_SCRATCH, nbytes, 1 << 20, "bias-gradient partials"), dout, rows, OC,
           groups, int(accumulate))
    return dbias_t


def encoder_fwd(tokens, wte, wpe, out=None):
    B, T = tokens.shape
    C = wte.shape[1]
    out = torch.empty(B, T, C, dtype=wte.dtype, device=wte.device) if out is None else out
    N.call("llmk_encoder_fwd", out, tokens, wte, wpe, B, T, C)
    return out


_BUCKETS: dict[tuple, tuple] = {}


def bucket_sort(tokens: torch.Tensor, max_token: int):
    """(sorted token ids, positions) of the flattened int32 ``tokens``, ordered by (token id, position): the
    framework's own stable radix sort on the device (no library sort, no allocation after the first call for a
    given size). The returned tensors are reused by the next call with the same number of tokens."""
    n = tokens.numel()
    key = (tokens.device.index, n)
    if key not in _BUCKETS:
        dev = tokens.device
        ints = int(N.lib().llmk_bucket_sort_scratch_ints(n))
        _BUCKETS[key] = (torch.empty(n, dtype=torch.int32, device=dev), torch.empty(n, dtype=torch.int32, device=dev),
                         torch.empty(ints, dtype=torch.int32, device=dev))
    st, sp, scratch = _BUCKETS[key]
    N.call("llmk_bucket_sort", st, sp, tokens, n, int(max_token), scratch)
    return st, sp


def encoder_bwd(dwte, dwpe, dout, tokens):
    """Deterministic: positions are bucketed by token id with a stable device sort, then each token's
    rows are summed in ascending position order."""
    B, T = tokens.shape
    C = dwte.shape[1]
    N.require_cuda_tensor(tokens, torch.int32, "tokens")
    sorted_tok, sorted_pos = bucket_sort(tokens, dwte.shape[0])
    N.call("llmk_encoder_bwd", dwte, dwpe, dout, sorted_tok, sorted_pos, B, T, C)
