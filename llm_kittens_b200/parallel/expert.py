"""Expert-parallel exchange for the mixture-of-experts model: symmetric (peer-mapped) buffers plus
the arrival tables that turn the dispatch / return kernels of ``csrc/moe.cu`` into an all-to-all.

A buffer allocated here exists on every rank at a known peer address, so a source rank stores its
routed rows directly into the owner's receive buffer. There is no barrier between the stages of a
layer: the dispatch kernel's last block release-stores the number of the exchange into the owners'
arrival tables (``arrival_table``), the expert GEMM's producer warp waits only for the entries of
the rows it is about to load, the return kernel publishes each (source, expert) block the same way
and the combine kernel waits for its owners inside the kernel. ``sync(tag)`` (a device-side barrier
over all ranks: signal + bounded wait) remains for set-up and tests. The library equivalent would be
one ``all_to_all_single`` per direction and layer (reference primitive: llmc/distributed_ext.cuh:27-48).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _native as N


class PeerExchange:
    def __init__(self, device: torch.device, group=None, timeout_ms: int | None = None):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.device = device
        self.group = group if group is not None else dist.group.WORLD
        self.world_size = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world_size > int(N.lib().llmk_comm_max_ranks()):
            raise RuntimeError("expert-parallel exchange serves at most 8 ranks of one NVLink domain")
        self.limit_ns = int((timeout_ms if timeout_ms is not None else int(os.environ.get("LLMK_PEER_TIMEOUT_MS", "30000"))) * 1e6)
        self._keep = []
        self.ctrl, self.ctrl_ptrs = self._alloc(int(N.lib().llmk_comm_ctrl_ints()), torch.int32)
        self.ctrl.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)
        self.epochs: dict[int, int] = {}

    def _alloc(self, numel: int, dtype):
        t = self._symm.empty(numel, dtype=dtype, device=self.device)
        hdl = self._symm.rendezvous(t, self.group)
        self._keep.append(hdl)
        ptrs = (ctypes.c_longlong * self.world_size)(*[int(p) for p in hdl.buffer_ptrs])
        return t, ptrs

    def alloc(self, numel: int, device=None):
        t, ptrs = self._alloc(numel, torch.bfloat16)
        t.zero_()
        return t, ptrs

    def arrival_table(self, entries: int, device=None):
        """Zeroed int32 table in symmetric memory + the host array of the ranks' pointers to it."""
        t, ptrs = self._alloc(entries, torch.int32)
        t.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        return t, ptrs

    def sync(self, tag: int) -> None:
        """All ranks' stores issued before this point are visible to every rank after it (device side)."""
        e = self.epochs.get(tag, 0) + 1
        self.epochs[tag] = e
        N.call("llmk_comm_signal", self.ctrl_ptrs, tag, self.rank, self.world_size, e)
        N.call("llmk_comm_wait", self.ctrl, tag, e, self.world_size, self.limit_ns, N.status_word())


class LibraryExchange:
    """The baseline the peer-memory exchange is measured against: the same dispatch / combine kernels, but rows travel
    through a packed send buffer and one ``torch.distributed.all_to_all_single`` (NCCL) per direction and layer, the
    collective the reference's primitive wraps (llmc/distributed_ext.cuh:27-48). The model checks ``library`` and takes
    the collective route; buffers are ordinary device tensors."""

    library = True
    limit_ns = int(2e9)

    def __init__(self, device: torch.device, group=None):
        self.device = device
        self.group = group if group is not None else dist.group.WORLD
        self.world_size = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)

    def alloc(self, numel: int, device=None):
        from ..ops import moe as moe_ops

        t = torch.zeros(numel, dtype=torch.bfloat16, device=self.device)
        return t, moe_ops.ptr_table([t])

    def arrival_table(self, entries: int, device=None):
        from ..ops import moe as moe_ops

        t = torch.zeros(entries, dtype=torch.int32, device=self.device)
        return t, moe_ops.ptr_table([t])

    def all_to_all(self, recv: torch.Tensor, send: torch.Tensor) -> None:
        dist.all_to_all_single(recv.view(-1), send.view(-1), group=self.group)

    def sync(self, tag: int) -> None:
        pass
