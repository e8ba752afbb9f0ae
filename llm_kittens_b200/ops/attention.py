"""Causal flash attention on packed QKV (``csrc/attention.cu``). Reference jobs:
llmc/attention.cuh:261-338, 481-604 and llmc/attention_gqa.cuh:415-572."""
from __future__ import annotations

import torch

from . import _native as N


import os

# "tc" = tcgen05/TMEM kernels (csrc/attention_tc.cu) where the shape allows, "warp" = warp-level MMA kernels
IMPL = os.environ.get("LLMK_ATTENTION", "tc")


def attention_fwd(qkv, B, T, NH, NKVH, HS, out=None, lse=None, impl=None):
    """``qkv``: [B, T, (NH+2*NKVH)*HS] -> ``out`` [B, T, NH*HS], ``lse`` [B, NH, T] fp32."""
    out = torch.empty(B, T, NH * HS, dtype=qkv.dtype, device=qkv.device) if out is None else out
    lse = torch.empty(B, NH, T, dtype=torch.float32, device=qkv.device) if lse is None else lse
    if (impl or IMPL) == "tc" and T % 128 == 0:
        N.call("llmk_attention_fwd_tc", out, lse, qkv, B, T, NH, NKVH, HS, N.status_word())
    else:
        N.call("llmk_attention_fwd", out, lse, qkv, B, T, NH, NKVH, HS)
    return out, lse


def fused_rope_available(T: int) -> bool:
    """Whether the tcgen05 kernels run for this sequence length, i.e. whether RoPE can live in the QKV GEMM's epilogue
    and its backward in the output tiles of the attention backward kernels."""
    return IMPL == "tc" and T % 128 == 0


def attention_bwd_prep(dout, out, dvec, B, T, NH, HS) -> bool:
    """D = rowsum(dO * O) into ``dvec`` [B, NH, T], the bandwidth-shaped first pass of the tcgen05 backward. A caller that
    runs it itself (e.g. on a side stream, beside a GEMM) passes ``prep_done=True`` to :func:`attention_bwd`. Returns
    False (and does nothing) when the warp-level fallback will run, which computes D inside its own entry point."""
    if IMPL == "tc" and T % 128 == 0:
        N.call("llmk_attention_bwd_prep", dvec, dout, out, B, T, NH, HS)
        return True
    return False


def attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS, dqkv=None, dvec=None, impl=None, rope=None, prep_done=False):
    """``rope`` ([T, HS/2, 2] table, tcgen05 path only): ``qkv`` holds rotated q / k and the dq / dk columns of ``dqkv``
    are returned as gradients of the un-rotated projections (the inverse rotation happens in the kernels' output tiles)."""
    dqkv = torch.empty_like(qkv) if dqkv is None else dqkv
    dvec = torch.empty(B, NH, T, dtype=torch.float32, device=qkv.device) if dvec is None else dvec
    if (impl or IMPL) == "tc" and T % 128 == 0:
        if not prep_done:
            N.call("llmk_attention_bwd_prep", dvec, dout, out, B, T, NH, HS)
        if rope is not None:
            N.call("llmk_attention_bwd_tc_rope", dqkv, dvec, dout, qkv, lse, B, T, NH, NKVH, HS, N.status_word(), rope)
        else:
            N.call("llmk_attention_bwd_tc", dqkv, dvec, dout, qkv, lse, B, T, NH, NKVH, HS, N.status_word())
    elif rope is not None:
        raise N.NativeError("attention_bwd: the fused RoPE backward needs the tcgen05 path (T a multiple of 128)")
    else:
        N.call("llmk_attention_bwd", dqkv, dvec, dout, qkv, out, lse, B, T, NH, NKVH, HS)
    return dqkv
