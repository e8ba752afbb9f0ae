"""tcgen05/TMEM GEMM family (``csrc/gemm_tcgen05.cu``).

* :func:`gemm_nt`  ``C[M,N] = A[M,K] @ B[N,K]^T``  (+bias, +GELU with pre-activation, +addend)
* :func:`gemm_nn`  ``C[M,N] = A[M,K] @ B[K,N]``    (optionally times GELU'(aux), or + addend)
* :func:`gemm_tn`  ``C[M,N] (+)= A[K,M]^T @ B[K,N]`` (split-K through an fp32 workspace; optionally the bias gradient
  ``dbias[M] (+)= A.sum(0)`` from the same launch, job of llmc/matmul.cuh:465-539)

They replace matmul_forward / matmul_forward_gelu / matmul_backward of the reference
(llmc/matmul.cuh:678-785, 1138-1201, 1238-1338).
"""
from __future__ import annotations

import os

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
    return N.scratch_buffer(_WORKSPACE, nbytes, 64 << 20, "split-K partials")


# Weights that another kernel is still filling while GEMMs already run on them (the tile-granular parameter gather of
# ZeRO-3, parallel/sharded.py): data pointer of the weight view -> [flags tensor, first flag, elements per flag, tick,
# time limit in ns]. A GEMM whose B operand is registered here polls the flags that cover each tile (llmk_gemm_b_ready).
_B_READY: dict[int, list] = {}


def register_b_ready(weight: torch.Tensor, flags: torch.Tensor, first_flag: int, chunk_elems: int, limit_ns: int) -> list:
    """Returns the registry entry; the owner of the gather sets ``entry[3]`` (the tick) before every gather and may set
    it to 0 to switch the polling off (flags are compared with ``>=``)."""
    entry = [flags[int(first_flag):], int(first_flag), int(chunk_elems), 0, int(limit_ns)]
    _B_READY[weight.data_ptr()] = entry
    return entry


def unregister_b_ready(weight: torch.Tensor) -> None:
    _B_READY.pop(weight.data_ptr(), None)


_TILE_ROWS = 0


def tile_rows() -> int:
    """Rows of C that one work unit of the kernel covers: 256 with CTA pairs, else 128."""
    global _TILE_ROWS
    if _TILE_ROWS == 0:
        _TILE_ROWS = 256 if int(N.lib().llmk_gemm_pair_clusters()) > 0 else 128
    return _TILE_ROWS


def _gemm(mode, epi, a, b, c, c2, bias, aux, M, Nn, K, groups=1, a_ready=None):
    """``M``, ``Nn``, ``K`` are the dimensions of ONE group; operands of a grouped call are stacked along their rows.
    ``a_ready`` = (int32 tensor, rows per entry, needed value, time limit in ns): the rows of A are still arriving and
    entry ``row // rows_per_entry`` tells when a block of them is complete (NT / NN only)."""
    for t, nm in ((a, "A"), (b, "B"), (c, "C")):
        N.require_cuda_tensor(t, torch.bfloat16, nm)
    if groups > 1 and (M % tile_rows() or (mode != MODE_NT and K % 64)):
        # a tile would straddle two groups: one launch per group on row slices of the stacked operands
        a_rows, b_rows = (K, K) if mode == MODE_TN else (M, Nn if mode == MODE_NT else K)
        for g in range(groups):
            cut = lambda t, r: None if t is None else t[g * r:(g + 1) * r]
            ar = None if a_ready is None else (a_ready[0][g * (M // a_ready[1]):], *a_ready[1:4])
            _gemm(mode, epi, cut(a, a_rows), cut(b, b_rows), cut(c, M), cut(c2, M), cut(bias, Nn) if bias is not None and bias.dim() == 1 else bias,
                  cut(aux, M), M, Nn, K, a_ready=ar)
        return c
    ws = None
    ws_bytes = 0
    if mode == MODE_TN:
        ws_bytes = int(N.lib().llmk_gemm_workspace_bytes(mode, M * groups, Nn, K, 0))
        if ws_bytes:
            ws = workspace(ws_bytes)
            ws_bytes = ws.numel()
    ready = _B_READY.get(b.data_ptr()) if (_B_READY and mode != MODE_TN) else None
    if a_ready is not None:
        if mode == MODE_TN or M % a_ready[1]:
            raise N.NativeError("gemm: a_ready needs an NT / NN product whose group rows are whole flag blocks")
        flags, rows_per, need, limit_ns = a_ready[:4]
        rotate = a_ready[4] if len(a_ready) > 4 else 0     # rows to start the walk at (a different source rank per rank)
        N.call("llmk_gemm_grouped_a_ready", mode, epi, a, b, c, c2, bias, aux, M, Nn, K, groups, ws, ws_bytes, N.status_word(),
               _MAX_CTAS, flags, rows_per, need, limit_ns, rotate)
    elif groups > 1:
        N.call("llmk_gemm_grouped", mode, epi, a, b, c, c2, bias, aux, M, Nn, K, groups, ws, ws_bytes, N.status_word(), _MAX_CTAS)
    elif ready is not None and ready[3] > 0:
        flags, first, chunk, tick, limit_ns = ready
        N.call("llmk_gemm_b_ready", mode, epi, a, b, c, c2, bias, aux, M, Nn, K, ws, ws_bytes, N.status_word(), _MAX_CTAS,
               flags, chunk, tick, limit_ns)
    else:
        N.call("llmk_gemm", mode, epi, a, b, c, c2, bias, aux, M, Nn, K, ws, ws_bytes, N.status_word(), _MAX_CTAS)
    return c


def _flat2(t, groups):
    """[G, R, C] (contiguous) -> [G*R, C]; 2-D tensors pass through."""
    if t is None or t.dim() == 2:
        return t
    assert t.is_contiguous()
    return t.view(-1, t.shape[-1])


def gemm_nt(a, b, bias=None, out=None, gelu_pre_out=None, add=None, groups=1, a_ready=None):
    """``out = a @ b.T (+ bias) (+ add)``; with ``gelu_pre_out`` the pre-activation goes there and
    ``out`` gets tanh-GELU of it. ``a``: [M,K], ``b``: [N,K].

    ``groups`` > 1: that many independent problems in one launch (the experts of an MoE layer): ``a`` [G*M,K],
    ``b`` [G,N,K] or [G*N,K], ``bias`` [G,N] or [G*N], ``out`` / ``gelu_pre_out`` / ``add`` [G*M,N]."""
    b = _flat2(b, groups)
    if bias is not None and bias.dim() == 2:
        bias = bias.reshape(-1)
    K = a.shape[1]
    M = a.shape[0] // groups
    Nn = b.shape[0] // groups
    assert b.shape[1] == K and a.shape[0] == M * groups and b.shape[0] == Nn * groups
    if out is None:
        out = torch.empty(M * groups, Nn, dtype=torch.bfloat16, device=a.device)
    epi = 0
    if bias is not None:
        epi |= EPI_BIAS
    if gelu_pre_out is not None:
        assert bias is not None and add is None
        epi |= EPI_GELU
    if add is not None:
        epi |= EPI_ADD
    return _gemm(MODE_NT, epi, a, b, out, gelu_pre_out, bias, add, M, Nn, K, groups, a_ready=a_ready)


def gemm_qkv_rope(a, w, rope, T, rope_cols, HS, out=None):
    """QKV projection with RoPE applied in the epilogue: ``out = a @ w.T`` ([M, (NH + 2*NKVH)*HS] packed q | k | v), the
    first ``rope_cols`` columns (q and k heads of ``HS`` columns) rotated by ``rope`` [T, HS/2, 2] (cos, sin of
    interleaved pairs) for token ``row % T`` before rounding; v is stored as is."""
    M, K = a.shape
    Nn = w.shape[0]
    for t, nm in ((a, "A"), (w, "B")):
        N.require_cuda_tensor(t, torch.bfloat16, nm)
    if out is None:
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device=a.device)
    ready = _B_READY.get(w.data_ptr()) if _B_READY else None
    if ready is not None and ready[3] > 0:
        flags, _, chunk, tick, limit_ns = ready
    else:
        flags, chunk, tick, limit_ns = None, 1, 0, 0
    N.call("llmk_gemm_qkv_rope", a, w, out, M, Nn, K, rope, T, rope_cols, HS, N.status_word(), _MAX_CTAS, flags, chunk, tick, limit_ns)
    return out


def gemm_swiglu(a, w_up, w_gate, act, up, gate) -> bool:
    """Llama MLP first half in one launch: ``up = a @ w_up.T``, ``gate = a @ w_gate.T``, ``act = silu(gate) * up`` with
    the SwiGLU in the GEMM's epilogue (all three [M, H] outputs are written). Returns False, having done nothing, when
    the shape or the device cannot take the fused kernel (H not a multiple of 128, no CTA pairs): the caller then runs
    two GEMMs and the stand-alone SwiGLU kernel."""
    M, K = a.shape
    H = w_up.shape[0]
    if H % 128 or K % 8 or tile_rows() != 256 or not hasattr(N.lib(), "llmk_gemm_swiglu"):
        return False
    for t, nm in ((a, "A"), (w_up, "W_up"), (w_gate, "W_gate"), (act, "act"), (up, "up"), (gate, "gate")):
        N.require_cuda_tensor(t, torch.bfloat16, nm)
    ru = _B_READY.get(w_up.data_ptr()) if _B_READY else None
    rg = _B_READY.get(w_gate.data_ptr()) if _B_READY else None
    if ru is not None and rg is not None and ru[3] > 0 and rg[3] > 0 and ru[2] == rg[2] and ru[3] == rg[3]:
        fu, fg, chunk, tick, limit_ns = ru[0], rg[0], ru[2], ru[3], ru[4]
    elif (ru is not None and ru[3] > 0) or (rg is not None and rg[3] > 0):
        return False          # weights still arriving with different flag geometries: take the unfused route
    else:
        fu = fg = None
        chunk, tick, limit_ns = 1, 0, 0
    N.call("llmk_gemm_swiglu", a, w_up, w_gate, act, up, gate, M, H, K, N.status_word(), _MAX_CTAS, fu, fg, chunk, tick, limit_ns)
    return True


def gemm_grouped_scatter(a, b, bias, shape_like, groups, dst_ptrs, arrive_ptrs, arrive_off, count, cap, P, rank, epoch, nn=False):
    """Second GEMM of a mixture-of-experts layer with the way back fused into its epilogue: ``a`` [G*P*cap, K] times the
    local experts' weights (``b`` [G, N, K] with ``bias`` [G, N], or with ``nn`` [G, K, N] and no bias); row
    (e_local, source rank, slot) of the result is stored into that source rank's buffer (``dst_ptrs``), and every
    completed (source rank, expert) block is published in the source rank's arrival table (``arrive_ptrs`` at
    ``arrive_off`` + expert index) with ``epoch``. ``count``: G*P zeroed int32; ``shape_like``: a local [G*P*cap, N]
    tensor that only lends its shape to a tensor map."""
    b2 = _flat2(b, groups)
    K = a.shape[1]
    M = a.shape[0] // groups
    Nn = b2.shape[1] if nn else b2.shape[0] // groups
    if bias is not None and bias.dim() == 2:
        bias = bias.reshape(-1)
    if M != P * cap or M % tile_rows() or (nn and K % 64):
        raise N.NativeError("gemm_grouped_scatter: expert row blocks must be whole tiles")
    N.call("llmk_gemm_grouped_scatter", MODE_NN if nn else MODE_NT, 0 if nn else 1, a, b2, shape_like, bias, M, Nn, K, groups,
           N.status_word(), _MAX_CTAS, dst_ptrs, arrive_ptrs, arrive_off, count, cap, P, rank, epoch)


def fused_drow_available(head_size: int) -> bool:
    """The input-gradient GEMM of the attention projection can also produce D = rowsum(dO * O) per head (head size 64:
    one epilogue chunk is one head; ``LLMK_FUSED_DROW=0`` turns it off)."""
    return head_size == 64 and hasattr(N.lib(), "llmk_gemm_nn_drow") and os.environ.get("LLMK_FUSED_DROW", "1") != "0"


def gemm_nn(a, b, out=None, dgelu_of=None, add=None, groups=1, a_ready=None, drow_of=None):
    """``out = a @ b`` with ``a``: [M,K], ``b``: [K,N]; optionally ``* gelu'(dgelu_of)`` or ``+ add``.
    ``groups`` > 1: ``a`` [G*M,K], ``b`` [G,K,N] or [G*K,N], ``out`` / aux [G*M,N].

    ``drow_of`` = (O [M,N], dvec [M/T, N/64, T] fp32, T): also ``dvec[b, h, t] = sum(out[b*T+t, 64h:64h+64] * O[...])``
    from the epilogue (the D term of the attention backward, with ``out`` = dO); returns False instead of the output,
    having done nothing, when the fused kernel cannot take the call (a weight that is still being gathered)."""
    b = _flat2(b, groups)
    K = a.shape[1]
    M = a.shape[0] // groups
    Nn = b.shape[1]
    assert b.shape[0] == K * groups and a.shape[0] == M * groups
    if out is None:
        out = torch.empty(M * groups, Nn, dtype=torch.bfloat16, device=a.device)
    if drow_of is not None:
        o, dvec, T = drow_of
        ready = _B_READY.get(b.data_ptr()) if _B_READY else None
        if groups != 1 or dgelu_of is not None or add is not None or Nn % 64 or M % T or (ready is not None and ready[3] > 0):
            return False
        for t, nm in ((a, "A"), (b, "B"), (out, "C"), (o, "O")):
            N.require_cuda_tensor(t, torch.bfloat16, nm)
        N.require_cuda_tensor(dvec, torch.float32, "dvec")
        assert o.numel() == M * Nn and dvec.numel() == M * (Nn // 64)
        N.call("llmk_gemm_nn_drow", a, b, out, o, dvec, M, Nn, K, T, Nn // 64, N.status_word(), _MAX_CTAS)
        return out
    epi = 0
    aux = None
    if dgelu_of is not None:
        epi, aux = EPI_DGELU, dgelu_of
    elif add is not None:
        epi, aux = EPI_ADD, add
    return _gemm(MODE_NN, epi, a, b, out, None, None, aux, M, Nn, K, groups, a_ready=a_ready)


def fused_dbias_available() -> bool:
    """The weight-gradient GEMM can also produce the bias gradient (CTA-pair kernel; ``LLMK_FUSED_DBIAS=0`` turns it off)."""
    return tile_rows() == 256 and hasattr(N.lib(), "llmk_gemm_tn_dbias") and os.environ.get("LLMK_FUSED_DBIAS", "1") != "0"


def gemm_tn(a, b, out=None, accumulate=False, groups=1, dbias=None):
    """``out (+)= a.T @ b`` with ``a``: [K,M], ``b``: [K,N] (K = token dimension).
    ``groups`` > 1: ``a`` [G*K,M], ``b`` [G*K,N], ``out`` [G,M,N] or [G*M,N]: group g uses rows [g*K,(g+1)*K).

    ``dbias`` [M] ([G, M] with groups): also ``dbias (+)= a.sum(0)`` per group (the bias gradient of the linear layer
    whose output gradient is ``a``), from the same launch when the fused kernel takes the call, else from the
    stand-alone column-sum kernel."""
    M = a.shape[1]
    K = a.shape[0] // groups
    Nn = b.shape[1]
    assert b.shape[0] == K * groups and a.shape[0] == K * groups
    if out is None:
        assert not accumulate
        out = torch.empty(M * groups, Nn, dtype=torch.bfloat16, device=a.device)
    out2 = _flat2(out, groups)
    fused = dbias is not None and fused_dbias_available() and dbias.data_ptr() % 16 == 0 and dbias.is_contiguous()
    if fused and groups > 1:      # stacked problems: whole tiles per group, as for every grouped launch
        fused = M % tile_rows() == 0 and K % 64 == 0 and hasattr(N.lib(), "llmk_gemm_grouped_tn_dbias")
    if fused:
        for t, nm in ((a, "A"), (b, "B"), (out2, "C"), (dbias, "dbias")):
            N.require_cuda_tensor(t, torch.bfloat16, nm)
        ws_bytes = int(N.lib().llmk_gemm_workspace_bytes(MODE_TN, M * groups, Nn, K, 0))
        ws = workspace(ws_bytes) if ws_bytes else None
        ws_n = ws.numel() if ws is not None else 0
        if groups == 1:
            N.call("llmk_gemm_tn_dbias", a, b, out2, dbias, int(accumulate), M, Nn, K, ws, ws_n, N.status_word(), _MAX_CTAS)
        else:
            N.call("llmk_gemm_grouped_tn_dbias", a, b, out2, dbias, int(accumulate), M, Nn, K, groups, ws, ws_n, N.status_word(),
                   _MAX_CTAS)
        return out
    _gemm(MODE_TN, EPI_ADD if accumulate else 0, a, b, out2, None, None, out2 if accumulate else None, M, Nn, K, groups)
    if dbias is not None:
        from . import elementwise as ew

        if groups == 1:
            ew.dbias(dbias, a, accumulate=accumulate)
        else:
            ew.dbias_grouped(dbias, a, groups, accumulate=accumulate)
    return out
