"""The fused communication kernels alone, against the NVLink rate:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m llm_kittens_b200.ops.bench_comm

For two bucket sizes (one GPT-2 124M block, 7.1 M parameters; one Llama-3 8B block, 218 M parameters) it times
``rs_bucket`` (reduce-scatter by peer loads + 1/P scale + norm partials), ``adamw_push`` (AdamW on the shard + bf16
stores into every rank's parameter buffer), ``ag_bucket`` (all-gather by peer loads) and ``ag_bucket_flags`` (the same
with per-chunk flags) with CUDA events after a barrier, takes the maximum over the ranks, and prints the bytes that
cross NVLink per GPU and direction divided by that time, beside the measured peer-copy rate of 770 GB/s per direction
(900 nominal). The NCCL collective of the same size is timed the same way for comparison.
"""
from __future__ import annotations

import ctypes
import os
import statistics
import sys

import torch
import torch.distributed as dist

from . import _native as N

LINK_MEASURED, LINK_NOMINAL = 770.0, 900.0


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    dist.init_process_group("nccl", device_id=dev)
    import torch.distributed._symmetric_memory as symm_mem

    from ..parallel.fused import comm_grid_x

    P = world
    keep = []

    def symmetric(numel, dtype):
        t = symm_mem.empty(numel, dtype=dtype, device=dev)
        h = symm_mem.rendezvous(t, dist.group.WORLD)
        keep.append(h)
        return t, (ctypes.c_longlong * P)(*[int(p) for p in h.buffer_ptrs])

    ctrl, ctrl_ptrs = symmetric(int(N.lib().llmk_comm_ctrl_ints()), torch.int32)
    ctrl.zero_()
    limit_ns = int(20e9)
    status = N.status_word()
    epoch = [0]

    def timed(fn, before=None, iters=5):
        samples = []
        for _ in range(iters + 2):
            if before is not None:
                before()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ms = torch.tensor([s.elapsed_time(e)], device=dev)
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            samples.append(float(ms.item()))
        return statistics.median(samples[2:])

    rows = []
    for label, tensors in (("GPT-2 124M block", [768 * 2304, 768 * 768, 768 * 3072, 3072 * 768]),
                           ("Llama-3 8B block", [4096 * 6144, 4096 * 4096, 4096 * 14336, 4096 * 14336, 14336 * 4096])):
        n = sum(tensors)
        grads, grad_ptrs = symmetric(n, torch.bfloat16)
        params, param_ptrs = symmetric(n, torch.bfloat16)
        grads.normal_(0, 0.01)
        params.normal_(0, 0.02)
        shard_n = n // P
        pshard, pshard_ptrs = symmetric(shard_n, torch.bfloat16)
        pshard.normal_(0, 0.02)
        gshard = torch.zeros(shard_n, dtype=torch.float32, device=dev)
        master, m, v = (torch.zeros(shard_n, dtype=torch.float32, device=dev) for _ in range(3))
        # segment tables as the communication classes build them: one row per tensor, this rank's slice
        rs_rows, ag_rows, adam_rows, flag_rows = [], [], [], []
        off = s_off = nflags = 0
        for size in tensors:
            ln = size // P
            rs_rows.append((off + rank * ln, s_off, ln))
            ag_rows.append((s_off, off, ln))
            adam_rows.append((off + rank * ln, s_off, ln, 1))
            cps = max(1, min(8, ln // (1 << 19)))
            while cps > 1 and ln % (cps * 8):
                cps -= 1
            flag_rows.append((s_off, off, ln, nflags, cps))
            nflags += P * cps
            off += size
            s_off += ln
        as_table = lambda r: torch.tensor(r, dtype=torch.int64, device=dev)
        rs_t, ag_t, adam_t, flag_t = as_table(rs_rows), as_table(ag_rows), as_table(adam_rows), as_table(flag_rows)
        gx = comm_grid_x(max(r[2] for r in rs_rows))
        partials = torch.zeros(len(rs_rows) * gx, dtype=torch.float32, device=dev)
        flags = torch.zeros(nflags, dtype=torch.int32, device=dev)
        arrivals = torch.zeros(nflags, dtype=torch.int32, device=dev)
        bpc = max(1, min(16, 600 // max(1, nflags)))
        scale = torch.ones(1, device=dev)
        max_cps = max(r[4] for r in flag_rows)

        def signal():
            epoch[0] += 1
            N.call("llmk_comm_signal", ctrl_ptrs, 0, rank, P, epoch[0])

        def rs():
            N.call("llmk_comm_rs_bucket", grad_ptrs, ctrl, 0, epoch[0], rs_t, len(rs_rows), gshard, partials, gx, P, 0, limit_ns, status)

        def push():
            N.call("llmk_comm_adamw_push", param_ptrs, master, gshard, m, v, adam_t, len(adam_rows), max(r[2] for r in adam_rows),
                   1e-4, 0.9, 0.95, 0.1, 0.05, 1e-8, 0.1, scale, 1234, P, rank)

        def ag():
            N.call("llmk_comm_ag_bucket", pshard_ptrs, params, ag_t, len(ag_rows), gx, P)

        tick = [0]

        def agf():
            tick[0] += 1
            N.call("llmk_comm_ag_bucket_flags", pshard_ptrs, params, flag_t, len(flag_rows), max_cps, P, flags, arrivals, bpc, tick[0])

        bytes_in = (P - 1) * shard_n * 2          # what one GPU pulls (rs, ag) or pushes (adamw_push) per direction
        t_rs = timed(rs, before=signal)
        t_push = timed(push)
        t_ag = timed(ag)
        t_agf = timed(agf)
        out = torch.empty(shard_n, dtype=torch.bfloat16, device=dev)
        t_nccl_rs = timed(lambda: dist.reduce_scatter_tensor(out, grads, op=dist.ReduceOp.AVG))
        t_nccl_ag = timed(lambda: dist.all_gather_into_tensor(params[: shard_n * P], out))
        for name, t in (("rs_bucket", t_rs), ("adamw_push", t_push), ("ag_bucket", t_ag), ("ag_bucket_flags", t_agf),
                        ("NCCL reduce_scatter", t_nccl_rs), ("NCCL all_gather", t_nccl_ag)):
            gbs = bytes_in / (t * 1e-3) / 1e9
            rows.append((label, n * 2 / 1e6, name, t, gbs, gx))
        del grads, params, pshard, gshard, master, m, v
    N.check_status()
    if rank == 0:
        print(f"# fused communication kernels on {P} GPUs: bytes per GPU and direction = (P-1)/P of the bucket; time = max over ranks")
        print(f"{'bucket':18s} {'MB':>8s} {'kernel':22s} {'grid_x':>6s} {'ms':>8s} {'GB/s/dir':>9s} {'of 770':>7s} {'of 900':>7s}")
        for label, mb, name, t, gbs, gx in rows:
            print(f"{label:18s} {mb:8.1f} {name:22s} {gx:6d} {t:8.3f} {gbs:9.1f} {gbs / LINK_MEASURED:7.2f} {gbs / LINK_NOMINAL:7.2f}")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
