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


def attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS, dqkv=None, dvec=None, impl=None):
    dqkv = torch.empty_like(qkv) if dqkv is None else dqkv
    dvec = torch.empty(B, NH, T, dtype=torch.float32, device=qkv.device) if dvec is None else dvec
    if (impl or IMPL) == "tc" and T % 128 == 0:
        N.call("llmk_attention_bwd_prep", dvec, dout, out, B, T, NH, HS)
        N.call("llmk_attention_bwd_tc", dqkv, dvec, dout, qkv, lse, B, T, NH, NKVH, HS, N.status_word())
    else:
        N.call("llmk_attention_bwd", dqkv, dvec, dout, qkv, out, lse, B, T, NH, NKVH, HS)
    return dqkv
