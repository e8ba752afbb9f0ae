"""Context-parallel (ring) causal attention on the framework's own kernels.

The sequence is split into P contiguous chunks; rank r holds positions [r*T, (r+1)*T) as a packed QKV tensor in
symmetric memory. Queries of rank r attend to the chunks 0..r: its own chunk causally, the earlier chunks in full.
Every step is one launch of the tcgen05 attention kernels whose key / value tiles are pulled straight out of the
owning rank's memory by TMA loads (``llmk_attention_fwd_ring_step`` / ``llmk_attention_bwd_ring_step``); with
NVSwitch every peer is one hop away, so no chunk is passed around a ring. The steps are folded together with their
log-sum-exp (forward) and summed (dQ); the dK / dV contributions that later ranks compute for a chunk stay in their
buffers until the chunk's owner sums them in rank order (deterministic). Job of the reference's ring attention local
step and its un-wired driver (llmc/tk/ring_attention_sm120.cuh:55-189, llmc/attention_ext.cuh). The library-level
implementation over ``torch.distributed`` in ``parallel/primitives.py`` is the CPU-testable counterpart.

Synchronisation is on the device: a signal / bounded-wait pair over a control buffer before peers' memory is read
(forward: the chunks are in place; backward: the contributions are in place) and at the end of the backward (nobody
still reads what the next call overwrites).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _native as N


class ContextParallelAttention:
    def __init__(self, B: int, T: int, NH: int, NKVH: int, HS: int, device: torch.device, group=None, timeout_ms: int | None = None):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        if T % 128 or HS not in (64, 128) or NH % NKVH:
            raise ValueError("context-parallel attention needs chunks of a multiple of 128 tokens and head size 64 or 128")
        self.group = group if group is not None else dist.group.WORLD
        self.P, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.P > int(N.lib().llmk_comm_max_ranks()):
            raise RuntimeError("context-parallel attention serves at most 8 ranks of one NVLink domain")
        self.B, self.T, self.NH, self.NKVH, self.HS = B, T, NH, NKVH, HS
        self.W = (NH + 2 * NKVH) * HS
        self.device = device
        self.limit_ns = int((timeout_ms if timeout_ms is not None else int(os.environ.get("LLMK_PEER_TIMEOUT_MS", "30000"))) * 1e6)
        self._keep = []

        def symmetric(numel, dtype):
            t = symm_mem.empty(numel, dtype=dtype, device=device)
            h = symm_mem.rendezvous(t, self.group)
            self._keep.append(h)
            return t, [int(p) for p in h.buffer_ptrs]

        n = B * T * self.W
        qkv, self.qkv_ptrs = symmetric(n, torch.bfloat16)
        self.qkv = qkv.view(B, T, self.W)                      # this rank's chunk; the QKV projection may write here
        contrib, contrib_ptrs = symmetric(self.P * n, torch.bfloat16)
        self.contrib = contrib.view(self.P, B, T, self.W)       # [chunk] = this rank's dK / dV contribution to that chunk
        self.contrib.zero_()
        # pointers to every rank's contribution buffer for MY chunk
        self.my_chunk_ptrs = (ctypes.c_longlong * self.P)(*[p + self.rank * n * 2 for p in contrib_ptrs])
        self.ctrl, ctrl_ptrs = symmetric(int(N.lib().llmk_comm_ctrl_ints()), torch.int32)
        self.ctrl.zero_()
        self.ctrl_ptrs = (ctypes.c_longlong * self.P)(*ctrl_ptrs)
        self.epoch = 0
        f32 = torch.float32
        self.out_step = torch.empty(B, T, NH * HS, dtype=torch.bfloat16, device=device)
        self.lse_step = torch.empty(B, NH, T, dtype=f32, device=device)
        self.out_acc = torch.empty(B, T, NH * HS, dtype=f32, device=device)
        self.lse = torch.empty(B, NH, T, dtype=f32, device=device)
        self.out = torch.empty(B, T, NH * HS, dtype=torch.bfloat16, device=device)
        self.dq_step = torch.empty(B, T, self.W, dtype=torch.bfloat16, device=device)
        self.dq_acc = torch.empty(B * T, NH * HS, dtype=f32, device=device)
        self.dvec = torch.empty(B, NH, T, dtype=f32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def _barrier(self) -> None:
        """Device-side: everything this rank queued so far is visible to the peers' kernels queued after their wait."""
        self.epoch += 1
        N.call("llmk_comm_signal", self.ctrl_ptrs, 0, self.rank, self.P, self.epoch)
        N.call("llmk_comm_wait", self.ctrl, 0, self.epoch, self.P, self.limit_ns, N.status_word())

    def forward(self, qkv: torch.Tensor | None = None) -> torch.Tensor:
        """``qkv`` [B, T, W] (or None when the caller already wrote ``self.qkv``) -> attention output [B, T, NH*HS]."""
        B, T, NH, NKVH, HS = self.B, self.T, self.NH, self.NKVH, self.HS
        if qkv is not None:
            self.qkv.copy_(qkv)
        self._barrier()
        for src in range(self.rank + 1):
            N.call("llmk_attention_fwd_ring_step", self.out_step, self.lse_step, self.qkv, ctypes.c_void_p(self.qkv_ptrs[src]), B, T, T,
                   NH, NKVH, HS, int(src == self.rank), N.status_word())
            N.call("llmk_attention_ring_merge", self.out_acc, self.lse, self.out_step, self.lse_step, B, T, NH, HS, int(src == 0))
        N.call("llmk_cast_f32_to_bf16", self.out, self.out_acc, self.out.numel())
        return self.out

    def backward(self, dout: torch.Tensor, dqkv: torch.Tensor | None = None) -> torch.Tensor:
        """Gradient of the last :meth:`forward` with respect to this rank's packed QKV chunk."""
        B, T, NH, NKVH, HS, W = self.B, self.T, self.NH, self.NKVH, self.HS, self.W
        dqkv = torch.empty(B, T, W, dtype=torch.bfloat16, device=self.device) if dqkv is None else dqkv
        rows, qc, kvc = B * T, NH * HS, 2 * NKVH * HS
        N.call("llmk_attention_bwd_prep", self.dvec, dout, self.out, B, T, NH, HS)
        for src in range(self.rank + 1):
            N.call("llmk_attention_bwd_ring_step", self.dq_step, self.contrib[src], self.dvec, dout, self.qkv,
                   ctypes.c_void_p(self.qkv_ptrs[src]), self.lse, B, T, T, NH, NKVH, HS, int(src == self.rank), N.status_word())
            N.call("llmk_ring_accumulate", self.dq_acc, self.dq_step, rows, W, 0, qc, int(src == 0))
        N.call("llmk_ring_store_cols", dqkv, self.dq_acc, rows, W, 0, qc)
        self._barrier()                                    # every rank's contributions are in place
        N.call("llmk_ring_sum_peers", dqkv, self.my_chunk_ptrs, rows, W, qc, kvc, self.rank, self.P)
        self._barrier()                                    # nobody reads a chunk or a contribution any more
        return dqkv
