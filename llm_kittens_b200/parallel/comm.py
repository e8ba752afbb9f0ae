"""Gradient / parameter communication back-ends for data-parallel training.

``LibraryComm`` issues ``torch.distributed`` collectives (NCCL on GPUs, gloo on CPU) per tensor
slice on a side stream, ordered after the compute stream by an event - the scheme of the reference
(multi_gpu_async_reduce_gradient, llmc/zero.cuh:623-668; parameter all-gather,
train_gpt2.cu:1362-1375). It is the measured baseline and the CPU-testable path.
``parallel/fused.py`` provides ``FusedComm``: the same interface implemented by the framework's own
kernels over NVLink peer memory, with the reduce-scatter fused into the norm / optimizer path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .zero import ZeroPlan


class SingleProcessComm:
    """No-op communication for one process."""

    world_size, rank = 1, 0
    fused = False

    def __init__(self, plan: ZeroPlan):
        self.plan = plan

    def reduce_bucket(self, grads: torch.Tensor, layer) -> None:
        pass

    def finish_reduce(self) -> None:
        pass

    def all_reduce_scalar(self, t: torch.Tensor, op: str = "sum") -> None:
        pass

    def gather_params(self, params: torch.Tensor) -> None:
        pass

    def barrier(self) -> None:
        pass


class LibraryComm:
    def __init__(self, plan: ZeroPlan, group=None, device: torch.device | None = None):
        self.plan = plan
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.fused = False
        self.device = device
        self.cuda = device is not None and device.type == "cuda"
        self.stream = torch.cuda.Stream(device=device) if self.cuda else None
        self._pending = []
        self._avg = dist.ReduceOp.AVG if self.cuda else dist.ReduceOp.SUM

    def _on_side_stream(self):
        if not self.cuda:
            import contextlib

            return contextlib.nullcontext()
        ev = torch.cuda.Event()
        ev.record()
        self.stream.wait_event(ev)
        return torch.cuda.stream(self.stream)

    def reduce_bucket(self, grads: torch.Tensor, layer) -> None:
        """Average the bucket's gradients over ranks: all-reduce (stage 0) or reduce-scatter into the
        owner's part of each slice (stage >= 1). Asynchronous with respect to the compute stream."""
        P = self.world_size
        with self._on_side_stream():
            for name, off, size in self.plan.layer_bucket(layer):
                full = grads[off: off + size]
                if not self.cuda:
                    # gloo: no reduce-scatter and no AVG; an all-reduce leaves the owner's part correct as well
                    dist.all_reduce(full, op=dist.ReduceOp.SUM, group=self.group)
                    full.div_(P)
                elif self.plan.sharded:
                    shard = size // P
                    out = full[self.rank * shard:(self.rank + 1) * shard]
                    dist.reduce_scatter_tensor(out, full, op=self._avg, group=self.group)
                else:
                    dist.all_reduce(full, op=self._avg, group=self.group)

    def finish_reduce(self) -> None:
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.stream)

    def all_reduce_scalar(self, t: torch.Tensor, op: str = "sum") -> None:
        if op == "avg":
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
            t.div_(self.world_size)
        else:
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)

    def gather_params(self, params: torch.Tensor) -> None:
        """After the sharded update: every rank broadcasts its part of every dense slice."""
        if not self.plan.sharded:
            return
        P = self.world_size
        for layer in [None] + list(range(self.plan.config.num_layers)):
            for name, off, size in self.plan.layer_bucket(layer):
                full = params[off: off + size]
                shard = size // P
                mine = full[self.rank * shard:(self.rank + 1) * shard]
                if self.cuda:
                    dist.all_gather_into_tensor(full, mine, group=self.group)
                else:
                    dist.all_gather([full[r * shard:(r + 1) * shard] for r in range(P)], mine.clone(), group=self.group)

    def gather_expert_params(self, params: torch.Tensor) -> None:
        """Expert-parallel tensors are updated by their owner only and are not part of ``gather_params``; training never
        reads another rank's experts, but a checkpoint's model file (written by rank 0) must hold all of them: every
        expert is broadcast from its owner. A collective; called when a checkpoint is written."""
        plan = self.plan
        if plan.P <= 1:
            return
        for slot in plan.layout.slots:
            if not slot.spec.expert:
                continue
            E = slot.spec.shape[0]
            per = slot.size // E
            for l in range(slot.layers):
                base = slot.offset + l * slot.size
                for e in range(E):
                    owner = plan._expert_owner(e, E)
                    src = owner if self.group is None else dist.get_global_rank(self.group, owner)
                    dist.broadcast(params[base + e * per: base + (e + 1) * per], src=src, group=self.group)

    def barrier(self) -> None:
        dist.barrier(group=self.group)
