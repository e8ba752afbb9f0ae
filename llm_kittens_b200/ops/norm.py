"""LayerNorm / RMSNorm forward (optionally fused with the preceding residual add) and backward
(``csrc/norm.cu``). Reference jobs: llmc/layernorm.cuh:527-584, llmc/rmsnorm.cuh:151-198."""
from __future__ import annotations

import torch

from . import _native as N

_SCRATCH: dict[int, torch.Tensor] = {}


def _scratch(nbytes: int) -> torch.Tensor:
    return N.scratch_buffer(_SCRATCH, nbytes, 1 << 20, "column-sum partials")


def layernorm_fwd(inp, weight, bias, out=None, mean=None, rstd=None):
    Nn, C = inp.shape
    out = torch.empty_like(inp) if out is None else out
    mean = torch.empty(Nn, dtype=torch.float32, device=inp.device) if mean is None else mean
    rstd = torch.empty(Nn, dtype=torch.float32, device=inp.device) if rstd is None else rstd
    N.call("llmk_layernorm_fwd", out, mean, rstd, inp, weight, bias, Nn, C)
    return out, mean, rstd


def residual_layernorm_fwd(inp1, inp2, weight, bias, residual=None, out=None, mean=None, rstd=None):
    """``residual = inp1 + inp2; out = LN(residual)``; ``residual`` may alias ``inp1``."""
    Nn, C = inp1.shape
    residual = torch.empty_like(inp1) if residual is None else residual
    out = torch.empty_like(inp1) if out is None else out
    mean = torch.empty(Nn, dtype=torch.float32, device=inp1.device) if mean is None else mean
    rstd = torch.empty(Nn, dtype=torch.float32, device=inp1.device) if rstd is None else rstd
    N.call("llmk_residual_layernorm_fwd", residual, out, mean, rstd, inp1, inp2, weight, bias, Nn, C)
    return residual, out, mean, rstd


def layernorm_bwd(dinp, dweight, dbias, dout, inp, weight, mean, rstd, accumulate_dinp=True):
    """``dinp (+)= dLN/dinp``, ``dweight += ``, ``dbias += `` (bf16 gradients, deterministic)."""
    Nn, C = inp.shape
    nbytes = int(N.lib().llmk_norm_bwd_scratch_bytes(Nn, C))
    N.call("llmk_layernorm_bwd", dinp, dweight, dbias, _scratch(nbytes), dout, inp, weight, mean, rstd, Nn, C,
           int(accumulate_dinp))
    return dinp


def rmsnorm_fwd(inp, weight, eps=1e-5, out=None, rstd=None):
    Nn, C = inp.shape
    out = torch.empty_like(inp) if out is None else out
    rstd = torch.empty(Nn, dtype=torch.float32, device=inp.device) if rstd is None else rstd
    N.call("llmk_rmsnorm_fwd", out, rstd, inp, weight, Nn, C, float(eps))
    return out, rstd


def residual_rmsnorm_fwd(inp1, inp2, weight, eps=1e-5, residual=None, out=None, rstd=None):
    Nn, C = inp1.shape
    residual = torch.empty_like(inp1) if residual is None else residual
    out = torch.empty_like(inp1) if out is None else out
    rstd = torch.empty(Nn, dtype=torch.float32, device=inp1.device) if rstd is None else rstd
    N.call("llmk_residual_rmsnorm_fwd", residual, out, rstd, inp1, inp2, weight, Nn, C, float(eps))
    return residual, out, rstd


def rmsnorm_bwd(dinp, dweight, dout, inp, weight, rstd, accumulate_dinp=True):
    Nn, C = inp.shape
    nbytes = int(N.lib().llmk_norm_bwd_scratch_bytes(Nn, C))
    N.call("llmk_rmsnorm_bwd", dinp, dweight, _scratch(nbytes), dout, inp, weight, rstd, Nn, C, int(accumulate_dinp))
    return dinp
