"""Fused data-parallel communication over NVLink peer memory (``csrc/comm_fused.cu``).

``FusedComm`` moves the model's gradient and parameter buffers into symmetric memory (every rank
maps every peer's copy; allocation and handle exchange go through
``torch.distributed._symmetric_memory``, the kernels are ours) and implements ZeRO >= 1 as

    backward of block l finished  -> ``signal`` (bucket l ready, release at system scope)
    side stream                   -> ``rs_bucket``: wait for all peers' flags, peer-load the P copies of
                                     this rank's shard, average in fp32, leave norm partials
    after the last bucket         -> ``norm_exchange``: scalar all-reduce through the control buffers,
                                     clip coefficient on the device
                                  -> ``adamw_push``: AdamW on the fp32 averaged shard, results stored
                                     into every rank's parameter buffer (the all-gather)
                                  -> ``signal`` (parameters ready); the next step waits for it.

The library collectives of ``parallel/comm.py`` are the baseline this is measured against and the
fallback when peer mapping is unavailable. Multicast (NVLS) binding is switched off: only plain peer
loads / stores are used.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _native as N
from .zero import ZeroPlan


def comm_grid_x(max_segment_elems: int) -> int:
    """Blocks per segment of the bucket kernels (``rs_bucket``, ``ag_bucket``): one per 256 KiB of the longest
    segment, at least 8 (enough for the 14 MB buckets of GPT-2 124M) and at most 64 (Llama-3 8B: 436 MB per block,
    ~390 blocks of 256 threads with up to eight 16-byte peer loads in flight per thread)."""
    return int(min(64, max(8, (max_segment_elems * 2) // (256 * 1024))))


class FusedComm:
    fused = True

    def __init__(self, plan: ZeroPlan, model, device: torch.device, timeout_ms: int | None = None):
        if plan.P < 2:
            raise RuntimeError("the fused path needs at least two ranks")
        # ZeRO-0 (replicated optimizer state): the same kernels with whole tensors as "shards": every rank peer-loads
        # and averages all P copies of every gradient (a one-shot all-reduce), holds the complete norm, and updates
        # all parameters in its own buffer; nothing is pushed.
        self.replicated = not plan.sharded
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.plan, self.model, self.device = plan, model, device
        self.world_size, self.rank = plan.P, plan.rank
        P = self.world_size
        if P > int(N.lib().llmk_comm_max_ranks()):
            raise RuntimeError(f"fused communication serves at most {N.lib().llmk_comm_max_ranks()} ranks")
        self.limit_ns = int((timeout_ms if timeout_ms is not None else int(os.environ.get("LLMK_PEER_TIMEOUT_MS", "30000"))) * 1e6)
        self.group = dist.group.WORLD
        n = model.num_parameters

        def symmetric(numel, dtype):
            t = symm_mem.empty(numel, dtype=dtype, device=device)
            hdl = symm_mem.rendezvous(t, self.group)
            ptrs = (ctypes.c_longlong * P)(*[int(p) for p in hdl.buffer_ptrs])
            return t, hdl, ptrs

        self.grads, self._gh, self.grad_ptrs = symmetric(n, torch.bfloat16)
        self.params, self._ph, self.param_ptrs = symmetric(n, torch.bfloat16)
        self.ctrl, self._ch, self.ctrl_ptrs = symmetric(int(N.lib().llmk_comm_ctrl_ints()), torch.int32)
        self.grads.zero_()
        self.ctrl.zero_()
        self.params.copy_(model.params)
        # the model now computes on the symmetric buffers
        model.params, model.grads = self.params, self.grads
        model.p, model.g = model.layout.views(self.params), model.layout.views(self.grads)
        torch.cuda.synchronize(device)
        dist.barrier()

        L = plan.config.num_layers
        self.slot_params, self.slot_norm = L + 1, L + 2
        self.epoch = 0
        # the same counter on the device: the bucket kernels read it when they run, so a micro-step recorded in a CUDA
        # graph can be replayed every step (the host bumps both copies in begin_step)
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=device)
        self.graph_capturable = True
        self.stream = torch.cuda.Stream(device=device)
        self.gshard = torch.zeros(plan.state_elements, dtype=torch.float32, device=device)
        # per-bucket segment tables (gradient offset of my slice, state offset, length)
        self.grid_x = comm_grid_x(max(s.length for s in plan.segments))
        self.buckets = {}
        base = 0
        by_key = {}
        for s in plan.segments:
            by_key.setdefault((s.tensor, s.layer), []).append(s)
        for layer in list(range(L)) + [None]:
            rows = []
            for name, off, size in plan.layer_bucket(layer):
                slot = plan.layout[name]
                lidx = layer if slot.spec.layered else 0
                for s in by_key[(name, lidx)]:
                    rows.append((s.param_off, s.state_off, s.length))
            table = torch.tensor(rows, dtype=torch.int64, device=device)
            self.buckets[layer] = (table, len(rows), base)
            base += len(rows) * self.grid_x
        # expert-parallel tensors are not reduced: their (already 1/P-scaled) local gradients are only
        # converted into the fp32 shard buffer, through the same kernel with a one-entry peer table
        lay = plan.layout
        erows = [(s.param_off, s.state_off, s.length) for s in plan.segments if lay[s.tensor].spec.expert]
        self.expert_table = torch.tensor(erows, dtype=torch.int64, device=device) if erows else None
        self.expert_base = base
        base += len(erows) * self.grid_x
        self.own_grad_ptr = (ctypes.c_longlong * 1)(int(self.grads.data_ptr()))
        self.own_param_ptr = (ctypes.c_longlong * 1)(int(self.params.data_ptr()))
        self.num_partials = base
        self.partials = torch.zeros(base, dtype=torch.float32, device=device)
        # optimizer table (parameter offset, state offset, length, decay flag)
        rows = [(s.param_off, s.state_off, s.length, int(s.decay)) for s in plan.segments]
        self.adam_segs = torch.tensor(rows, dtype=torch.int64, device=device)
        self.adam_max_len = max(r[2] for r in rows)
        self._event = torch.cuda.Event()

    # ------------------------------------------------------------------ step protocol
    def begin_step(self) -> None:
        """Before gradients are zeroed: every peer must have finished reading last step's gradients and
        pushing its parameter shard (both are implied by its "parameters ready" flag)."""
        if self.epoch > 0:
            N.call("llmk_comm_wait", self.ctrl, self.slot_params, self.epoch, self.world_size, self.limit_ns, N.status_word())
        self.epoch += 1
        self.epoch_dev.add_(1)

    def reduce_bucket(self, grads: torch.Tensor, layer) -> None:
        slot = self.plan.config.num_layers if layer is None else layer
        N.call("llmk_comm_signal_dev", self.ctrl_ptrs, slot, self.rank, self.world_size, self.epoch_dev)
        self._event.record()
        self.stream.wait_event(self._event)
        table, nseg, base = self.buckets[layer]
        with torch.cuda.stream(self.stream):
            N.call("llmk_comm_rs_bucket_dev", self.grad_ptrs, self.ctrl, slot, self.epoch_dev, table, nseg, self.gshard,
                   self.partials[base:], self.grid_x, self.world_size, 0, self.limit_ns, N.status_word())

    def join_buckets(self) -> None:
        """The current stream waits for the bucket kernels queued so far (the end of a captured micro-step: every
        stream that forked from the capturing stream has to come back to it)."""
        torch.cuda.current_stream().wait_stream(self.stream)

    def finish_reduce(self) -> None:
        if self.expert_table is not None:
            # epoch 0 is always satisfied: no peer is involved in this copy
            N.call("llmk_comm_rs_bucket", self.own_grad_ptr, self.ctrl, 0, 0, self.expert_table, int(self.expert_table.shape[0]),
                   self.gshard, self.partials[self.expert_base:], self.grid_x, 1, 0, self.limit_ns, N.status_word())
        torch.cuda.current_stream().wait_stream(self.stream)

    def norm_and_clip(self, clip: float, scale: torch.Tensor, norm: torch.Tensor, flag: torch.Tensor,
                      loss: torch.Tensor | None = None) -> None:
        """Global gradient norm and clip coefficient; ``loss`` (one float, this rank's mean loss) comes back as the mean
        over the ranks from the same exchange, so a step has no library all-reduce."""
        N.call("llmk_comm_norm_exchange", self.ctrl_ptrs, self.partials, self.num_partials, self.slot_norm, self.rank,
               self.world_size, self.epoch, float(clip), scale, norm, flag, loss,
               1.0 / self.world_size if self.replicated else 1.0, self.limit_ns, N.status_word())

    def adamw_push(self, master, m, v, lr, beta1, beta2, step, eps, wd, scale, seed) -> None:
        b1c, b2c = 1.0 - beta1 ** step, 1.0 - beta2 ** step
        # replicated state: every rank updates everything in its own buffer (a one-entry peer table)
        ptrs, P, me = (self.own_param_ptr, 1, 0) if self.replicated else (self.param_ptrs, self.world_size, self.rank)
        N.call("llmk_comm_adamw_push", ptrs, master, self.gshard, m, v, self.adam_segs, int(self.adam_segs.shape[0]),
               self.adam_max_len, float(lr), float(beta1), float(beta2), float(b1c), float(b2c), float(eps), float(wd), scale,
               int(seed) & 0xFFFFFFFF, P, me)
        N.call("llmk_comm_signal", self.ctrl_ptrs, self.slot_params, self.rank, self.world_size, self.epoch)

    def skip_update(self) -> None:
        """A step whose update is skipped still has to tell the peers that this rank is done with the step: the
        "parameters ready" flag is what the next ``begin_step`` of every rank waits for before it zeroes the
        gradients that peers read. Queued after ``norm_and_clip``, it is ordered after every rank's gradient reads."""
        N.call("llmk_comm_signal", self.ctrl_ptrs, self.slot_params, self.rank, self.world_size, self.epoch)

    # ------------------------------------------------------------------ library-style helpers
    def all_reduce_scalar(self, t: torch.Tensor, op: str = "sum") -> None:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        if op == "avg":
            t.div_(self.world_size)

    def gather_params(self, params: torch.Tensor) -> None:
        """Parameter shards that were written locally only (e.g. after a resume): broadcast them."""
        P = self.world_size
        for layer in [None] + list(range(self.plan.config.num_layers)):
            for name, off, size in self.plan.layer_bucket(layer):
                full = params[off: off + size]
                shard = size // P
                dist.all_gather_into_tensor(full, full[self.rank * shard:(self.rank + 1) * shard].clone(), group=self.group)

    def barrier(self) -> None:
        dist.barrier(group=self.group)
