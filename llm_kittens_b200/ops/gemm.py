"""tcgen05/TMEM GEMM family (``csrc/gemm_tcgen05.cu``).

* :func:`gemm_nt`  ``C[M,N] = A[M,K] @ B[N,K]^T``  (+bias, +GELU with pre-activation, +addend)
* :func:`gemm_nn`  ``C[M,N] = A[M,K] @ B[K,N]``    (optionally times GELU'(aux), or + addend)
* :func:`gemm_tn`  ``C[M,N] (+)= A[K,M]^T @ B[K,N]`` (split-K through an fp32 workspace)

They replace matmul_forward / matmul_forward_gelu / matmul_backward of the reference
(llmc/matmul.cuh:678-785, 1138-1201, 1238-1338).
"""
from __future__ import annotations

import torch

from . import _native as N

MODE_NT, MODE_NN, MODE_TN = 0, 1, 2
EPI_BIAS, EPI_GELU, EPI_DGELU, EPI_ADD = 1, 2, 4, 8

_WORKSPACE: dict[int, torch.Tensor] = {}
_MAX_CTAS = 0  # 0 = one CTA per SM


def set_max_ctas(n: int) -> None:
    """Limit the persistent grid (used when a communication kernel needs SMs of its own)."""
    global _MAX_CTAS
    _MAX_CTAS = int(n)


def workspace(nbytes: int) -> torch.Tensor:
    dev = torch.cuda.current_device()
    ws = _WORKSPACE.get(dev)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 64 << 20), dtype=torch.uint8, device=f"cuda:{dev}")
        _WORKSPACE[dev] = ws
    return ws


def _gemm(mode, epi, a, b, c, c2, bias, aux, M, Nn, K):
    for t, nm in ((a, "A"), (b, "B"), (c, "C")):
        N.require_cuda_tensor(t, torch.bfloat16, nm)
    ws = None
    ws_bytes = 0
    if mode == MODE_TN:
        ws_bytes = int(N.lib().llmk_gemm_workspace_bytes(mode, M, Nn, K, 0))
        if ws_bytes:
            ws = workspace(ws_bytes)
            ws_bytes = ws.numel()
    N.call("llmk_gemm", mode, epi, a, b, c, c2, bias, aux, M, Nn, K, ws, ws_bytes, N.status_word(), _MAX_CTAS)
    return c


def gemm_nt(a, b, bias=None, out=None, gelu_pre_out=None, add=None):
    """``out = a @ b.T (+ bias) (+ add)``; with ``gelu_pre_out`` the pre-activation goes there and
    ``out`` gets tanh-GELU of it. ``a``: [M,K], ``b``: [N,K]."""
    M, K = a.shape
    Nn = b.shape[0]
    assert b.shape[1] == K
    if out is None:
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device=a.device)
    epi = 0
    if bias is not None:
        epi |= EPI_BIAS
    if gelu_pre_out is not None:
        assert bias is not None and add is None
        epi |= EPI_GELU
    if add is not None:
        epi |= EPI_ADD
    return _gemm(MODE_NT, epi, a, b, out, gelu_pre_out, bias, add, M, Nn, K)


def gemm_nn(a, b, out=None, dgelu_of=None, add=None):
    """``out = a @ b`` with ``a``: [M,K], ``b``: [K,N]; optionally ``* gelu'(dgelu_of)`` or ``+ add``."""
    M, K = a.shape
    Nn = b.shape[1]
    assert b.shape[0] == K
    if out is None:
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device=a.device)
    epi = 0
    aux = None
    if dgelu_of is not None:
        epi, aux = EPI_DGELU, dgelu_of
    elif add is not None:
        epi, aux = EPI_ADD, add
    return _gemm(MODE_NN, epi, a, b, out, None, None, aux, M, Nn, K)


def gemm_tn(a, b, out=None, accumulate=False):
    """``out (+)= a.T @ b`` with ``a``: [K,M], ``b``: [K,N] (K = token dimension)."""
    K, M = a.shape
    Nn = b.shape[1]
    assert b.shape[0] == K
    if out is None:
        assert not accumulate
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device=a.device)
    return _gemm(MODE_TN, EPI_ADD if accumulate else 0, a, b, out, None, None, out if accumulate else None, M, Nn, K)
