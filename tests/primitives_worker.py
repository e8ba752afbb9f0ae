"""Worker for tests/test_primitives_cpu.py: argv = mode out_dir; gloo ranks on CPU."""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from llm_kittens_b200.parallel import primitives as P  # noqa: E402


def main():
    mode, out_dir = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    g = torch.Generator().manual_seed(7)
    res = {}
    if mode == "tp":
        x = torch.randn(6, 16, generator=g)
        w1, b1 = torch.randn(32, 16, generator=g), torch.randn(32, generator=g)
        w2 = torch.randn(16, 32, generator=g)
        dy = torch.randn(6, 16, generator=g)
        # column-parallel up projection followed by row-parallel down projection (the Megatron MLP split)
        w1s, b1s, w2s = P.tp_slice_columns(w1, rank, world), b1.chunk(world)[rank], P.tp_slice_rows(w2, rank, world)
        h = P.column_parallel_forward(x, w1s, b1s)
        y = P.row_parallel_forward(h, w2s)
        dh, dw2s = P.row_parallel_backward(dy, h, w2s)
        dx, dw1s, db1s = P.column_parallel_backward(dh, x, w1s)
        res = dict(y=y, dx=dx, dw1s=dw1s, db1s=db1s, dw2s=dw2s)
    elif mode == "sp":
        full = torch.randn(2, 8, 4, generator=g)
        shard = full.chunk(world, dim=1)[rank].contiguous()
        gathered = P.sp_all_gather(shard)
        back = P.sp_reduce_scatter(gathered)          # every rank contributes the same tensor: world * shard
        a2a = P.all_to_all_equal(torch.arange(world * 2, dtype=torch.float32) + 100 * rank)
        res = dict(gathered=gathered, back=back, a2a=a2a, full=full)
    elif mode == "pp":
        torch.manual_seed(3)
        stages = [torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Tanh()) for _ in range(world)]
        micro = [torch.randn(4, 8, generator=g) for _ in range(5)]
        targets = [torch.randn(4, 8, generator=g) for _ in range(5)]
        mod = stages[rank]
        loss = P.run_pipeline(mod, micro if rank == 0 else targets, lambda y, t: ((y - t) ** 2).mean(), (4, 8))
        res = dict(loss=loss, grads=[p.grad.clone() for p in mod.parameters()])
        if rank == 0:   # single-process reference of the whole pipeline
            torch.manual_seed(3)
            ref = [torch.nn.Sequential(torch.nn.Linear(8, 8), torch.nn.Tanh()) for _ in range(world)]
            tot = 0.0
            for x, t in zip(micro, targets):
                y = x
                for s in ref:
                    y = s(y)
                l = ((y - t) ** 2).mean()
                l.backward()
                tot += float(l)
            res["ref_loss"] = tot
            res["ref_grads"] = [[p.grad.clone() for p in s.parameters()] for s in ref]
    elif mode == "ring":
        B, H, S, D = 2, 3, 8 * world, 16
        q, k, v = (torch.randn(B, H, S, D, generator=g) for _ in range(3))
        dout = torch.randn(B, H, S, D, generator=g)
        sl = slice(rank * 8, (rank + 1) * 8)
        ql, kl, vl = (t[:, :, sl].clone().requires_grad_(True) for t in (q, k, v))
        out = P.ring_attention(ql, kl, vl)
        out.backward(dout[:, :, sl])
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=True)
        ref.backward(dout)
        res = dict(out=out.detach(), ref=ref.detach()[:, :, sl], dq=ql.grad, dk=kl.grad, dv=vl.grad, rdq=qf.grad[:, :, sl],
                   rdk=kf.grad[:, :, sl], rdv=vf.grad[:, :, sl])
    elif mode == "experts":
        # expert-parallel parameters before a checkpoint: every rank holds its own experts' values (rank + 1) and stale
        # values (-1) for the others; after the gather every rank holds every owner's values, dense tensors untouched
        from llm_kittens_b200.models.config import ModelConfig
        from llm_kittens_b200.parallel.comm import LibraryComm
        from llm_kittens_b200.parallel.zero import ZeroPlan

        cfg = ModelConfig(family="moe", max_seq_len=128, vocab_size=512, padded_vocab_size=512, num_layers=2, num_heads=2,
                          num_kv_heads=2, channels=64, hidden_dim=128, num_experts=4, top_k=2)
        plan = ZeroPlan(cfg, world, rank, 1)
        params = torch.full((plan.layout.total,), -1.0, dtype=torch.bfloat16)
        owner_of = torch.full((plan.layout.total,), -1.0)
        for slot in plan.layout.slots:
            if slot.spec.expert:
                E = slot.spec.shape[0]
                per = slot.size // E
                for l in range(slot.layers):
                    for e in range(E):
                        lo = slot.offset + l * slot.size + e * per
                        o = plan._expert_owner(e, E)
                        owner_of[lo:lo + per] = o + 1
                        if o == rank:
                            params[lo:lo + per] = rank + 1
            else:
                params[slot.offset: slot.offset + slot.total] = 7.0
                owner_of[slot.offset: slot.offset + slot.total] = 7.0
        LibraryComm(plan).gather_expert_params(params)
        res = dict(params=params.float(), want=owner_of, experts=sum(s.total for s in plan.layout.slots if s.spec.expert))
    torch.save(res, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
