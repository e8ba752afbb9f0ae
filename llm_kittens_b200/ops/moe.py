"""Mixture-of-experts routing / dispatch / combine kernels (``csrc/moe.cu``). Semantics of the
reference's primitives llmc/moe.cuh:40-335 (top-k softmax routing, capacity dropping, permute /
unpermute), llmc/distributed_ext.cuh:27-48 (equal-split all-to-all) and llmc/losses.cuh:522-559
(load-balance loss), with deterministic slot assignment and peer-memory dispatch."""
from __future__ import annotations

import ctypes

import torch

from . import _native as N


def ptr_table(tensors_or_ptrs) -> ctypes.Array:
    """Host array of device pointers (one per rank) from tensors or raw integer addresses."""
    vals = [int(t.data_ptr()) if isinstance(t, torch.Tensor) else int(t) for t in tensors_or_ptrs]
    return (ctypes.c_longlong * len(vals))(*vals)


def router_fwd(x, wr, K, probs=None, top_idx=None, top_w=None):
    Nn, C = x.shape
    E = wr.shape[0]
    dev = x.device
    probs = torch.empty(Nn, E, dtype=torch.float32, device=dev) if probs is None else probs
    top_idx = torch.empty(Nn, K, dtype=torch.int32, device=dev) if top_idx is None else top_idx
    top_w = torch.empty(Nn, K, dtype=torch.float32, device=dev) if top_w is None else top_w
    N.call("llmk_moe_router_fwd", probs, top_idx, top_w, x, wr, Nn, C, E, K)
    return probs, top_idx, top_w


def assign_slots(top_idx, E, cap, slot=None, counts=None):
    Nn, K = top_idx.shape
    slot = torch.empty(Nn, K, dtype=torch.int32, device=top_idx.device) if slot is None else slot
    counts = torch.empty(E, dtype=torch.int32, device=top_idx.device) if counts is None else counts
    N.call("llmk_moe_assign_slots", slot, counts, top_idx, Nn, K, E, cap)
    return slot, counts


def dispatch(recv_ptrs, x, top_idx, slot, top_w, counts, E, cap, rank=0, P=1, scale_by_weight=False):
    Nn, K = top_idx.shape
    N.call("llmk_moe_dispatch", recv_ptrs, x, top_idx, slot, top_w, counts, Nn, K, x.shape[1], E, cap, rank, P, int(scale_by_weight))


def dispatch_signal(recv_ptrs, x, top_idx, slot, top_w, counts, E, cap, rank, P, scale_by_weight, arrive_ptrs, arrive_off, done, epoch):
    """:func:`dispatch` whose last block release-stores ``epoch`` into entry ``arrive_off + e_local * P + rank`` of the
    owner of every expert (``arrive_ptrs``: the ranks' arrival tables; ``done``: one zeroed int32 of local scratch)."""
    Nn, K = top_idx.shape
    N.call("llmk_moe_dispatch_signal", recv_ptrs, x, top_idx, slot, top_w, counts, Nn, K, x.shape[1], E, cap, rank, P,
           int(scale_by_weight), arrive_ptrs, arrive_off, done, epoch)


def return_signal(back_ptrs, y, C, E, cap, rank, P, arrive_ptrs, arrive_off, done, epoch):
    """:func:`return_rows` that publishes every (source rank, local expert) block with a release store of ``epoch`` into
    entry ``arrive_off + e`` of the source rank's arrival table (``done``: ``E/P * P`` zeroed int32 of local scratch)."""
    N.call("llmk_moe_return_signal", back_ptrs, y, C, E, cap, rank, P, arrive_ptrs, arrive_off, done, epoch)


def combine_wait(out, base, back, top_idx, slot, weights, cap, returned, E, epoch, limit_ns):
    """:func:`combine` that first waits inside the kernel (bounded) until ``returned[0:E]`` all hold ``epoch``."""
    Nn, K = top_idx.shape
    N.call("llmk_moe_combine_wait", out, base, back, top_idx, slot, weights, Nn, K, out.shape[1], cap, returned, E, epoch, limit_ns,
           N.status_word())
    return out


def inverse_map(inv_tok, inv_w, top_idx, slot, top_w, E, cap):
    """Source side of the pull-style dispatch: ``inv_tok[e*cap + s]`` = token that holds slot ``s`` of expert ``e`` (-1:
    unused), ``inv_w`` its routing weight; both in peer-readable memory."""
    Nn, K = top_idx.shape
    N.call("llmk_moe_inverse_map", inv_tok, inv_w, top_idx, slot, top_w, Nn, K, E, cap)


def source_ready(arrive_ptrs, arrive_off, E, rank, P, epoch):
    """This rank's token rows and maps are in place: entry ``arrive_off + E + rank`` of every rank's table gets ``epoch``."""
    N.call("llmk_moe_source_ready", arrive_ptrs, arrive_off, E, rank, P, epoch)


def dispatch_pull(recv, x_ptrs, tok_ptrs, w_ptrs, C, E, cap, rank, P, scale_by_weight, ready, done, epoch, limit_ns):
    """Owner side: fill ``recv`` [e_local][source][slot][C] by peer loads from the sources' rows and maps; waits per source
    for its ``source_ready``, publishes every finished (source, expert) block in ``ready[e_local*P + source]``."""
    N.call("llmk_moe_dispatch_pull", recv, x_ptrs, tok_ptrs, w_ptrs, C, E, cap, rank, P, int(scale_by_weight), ready, done, epoch,
           limit_ns, N.status_word())


def publish(arrive_ptrs, arrive_off, E, rank, P, epoch):
    """Owner side of the pull-style way back: after everything queued so far (the second expert GEMM), entry
    ``arrive_off + e`` of every rank's arrival table gets ``epoch`` for each expert ``e`` of this rank."""
    N.call("llmk_moe_publish", arrive_ptrs, arrive_off, E, rank, P, epoch)


def combine_pull(out, base, y_ptrs, save, top_idx, slot, weights, E, cap, rank, P, returned, epoch, limit_ns):
    """:func:`combine` whose rows are fetched from the owners' expert-output buffers (``y_ptrs``: the ranks' buffers laid
    out [e_local][source rank][slot]) by peer loads, after an in-kernel wait for the owners' ``publish``; ``save``
    (optional [E*cap, C]) keeps the fetched rows locally."""
    Nn, K = top_idx.shape
    N.call("llmk_moe_combine_pull", out, base, y_ptrs, save, top_idx, slot, weights, Nn, K, out.shape[1], E, cap, rank, P, returned,
           epoch, limit_ns, N.status_word())
    return out


def return_rows(back_ptrs, y, C, E, cap, rank=0, P=1):
    N.call("llmk_moe_return", back_ptrs, y, C, E, cap, rank, P)


def combine(out, base, back, top_idx, slot, weights, cap):
    Nn, K = top_idx.shape
    N.call("llmk_moe_combine", out, base, back, top_idx, slot, weights, Nn, K, out.shape[1], cap)
    return out


def combine_dweight(dout, back, top_idx, slot, cap, dw=None):
    Nn, K = top_idx.shape
    dw = torch.empty(Nn, K, dtype=torch.float32, device=dout.device) if dw is None else dw
    N.call("llmk_moe_combine_dweight", dw, dout, back, top_idx, slot, Nn, K, dout.shape[1], cap)
    return dw


def density(probs, coef, dens=None, aux_loss=None, accumulate=False):
    Nn, E = probs.shape
    dens = torch.empty(E, dtype=torch.float32, device=probs.device) if dens is None else dens
    aux_loss = torch.zeros(1, dtype=torch.float32, device=probs.device) if aux_loss is None else aux_loss
    N.call("llmk_moe_density", dens, aux_loss, probs, Nn, E, float(coef), int(accumulate))
    return dens, aux_loss


def router_bwd(probs, top_idx, top_w, dw, slot, dens, aux_scale, dlogits=None):
    Nn, E = probs.shape
    K = top_idx.shape[1]
    Epad = (E + 7) // 8 * 8
    dlogits = torch.empty(Nn, Epad, dtype=torch.bfloat16, device=probs.device) if dlogits is None else dlogits
    N.call("llmk_moe_router_bwd", dlogits, probs, top_idx, top_w, dw, slot, dens, Nn, E, Epad, K, float(aux_scale))
    return dlogits
