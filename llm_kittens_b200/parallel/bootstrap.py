"""Process-group bootstrap and communication back-end selection.

One process per GPU. Rendezvous goes through ``torch.distributed`` (NCCL on GPUs, gloo on CPU): from
the environment set by ``torch.distributed.run`` or from the trainer flags ``-pi tcp|fs|mpi``,
``-ps <server ip>``, ``-pf <shared path>``, ``-pn``, ``-pr`` (the reference's own rendezvous code is
llmc/zero.cuh:229-466). ``make_comm`` picks the fused NVLink kernels when the job has more than one
GPU and peer memory is available, and the library collectives otherwise.
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

from .comm import LibraryComm, SingleProcessComm
from .zero import ZeroPlan


def init_process_group(num_processes: int, rank: int, init_method: str = "env", server_ip: str = "", fs_path: str = "",
                       device: torch.device | None = None, timeout_s: int = 600) -> None:
    """``init_method``: ``env`` (torch.distributed.run), ``tcp`` (rank 0 listens on ``server_ip``:12345),
    ``fs`` (shared file under ``fs_path``) or ``mpi`` (ranks from OMPI_* variables, TCP rendezvous)."""
    if dist.is_initialized():
        return
    backend = "nccl" if device is not None and device.type == "cuda" else "gloo"
    kw = dict(backend=backend, timeout=datetime.timedelta(seconds=timeout_s))
    if backend == "nccl":
        kw["device_id"] = device
    if init_method == "env":
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "12345")
        dist.init_process_group(rank=rank, world_size=num_processes, **kw)
    elif init_method == "tcp":
        dist.init_process_group(init_method=f"tcp://{server_ip or '127.0.0.1'}:12345", rank=rank, world_size=num_processes, **kw)
    elif init_method == "fs":
        if not fs_path:
            raise ValueError("-pf <shared directory> is required with -pi fs")
        dist.init_process_group(init_method=f"file://{os.path.join(fs_path, 'llmk_rendezvous.sync')}", rank=rank,
                                world_size=num_processes, **kw)
    elif init_method == "mpi":
        rank = int(os.environ.get("OMPI_COMM_WORLD_RANK", rank))
        num_processes = int(os.environ.get("OMPI_COMM_WORLD_SIZE", num_processes))
        dist.init_process_group(init_method=f"tcp://{server_ip or os.environ.get('MASTER_ADDR', '127.0.0.1')}:12345", rank=rank,
                                world_size=num_processes, **kw)
    else:
        raise ValueError(f"unknown init method {init_method}")


def make_comm(plan: ZeroPlan, model, world: int, rank: int, device: torch.device, prefer: str = "auto"):
    """Communication back-end for a trainer: ``auto`` = fused kernels on multi-GPU CUDA jobs, else library."""
    if world == 1:
        return SingleProcessComm(plan)
    if prefer in ("auto", "fused") and device.type == "cuda":
        try:
            if plan.stage >= 2 and not plan._has_experts():
                from .sharded import ShardedComm

                return ShardedComm(plan, model, device)   # gradients (and parameters) really sharded
            from .fused import FusedComm

            return FusedComm(plan, model, device)
        except Exception as e:  # peer memory not available: fall back loudly
            if prefer == "fused":
                raise
            if rank == 0:
                print(f"[llm_kittens_b200] fused communication unavailable ({e}); using library collectives")
    return LibraryComm(plan, group=None, device=device)
