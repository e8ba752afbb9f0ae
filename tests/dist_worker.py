"""Worker process for the multi-rank tests (spawned by test_dist_cpu.py / test_dist_gpu.py).

argv: mode out_dir  (rank / world / rendezvous come from the environment set by the test).
modes:
  cpu_zero<k>      gloo, PyTorch oracle model in fp32, ZeRO stage k, library collectives
  gpu_library<k>   NCCL, CUDA model, ZeRO stage k, library collectives
  gpu_fused        NCCL bootstrap, CUDA model, ZeRO-1 through the fused peer-memory kernels
  gpu_fused0       the same kernels with replicated optimizer state (ZeRO-0: one-shot all-reduce by peer loads)
  gpu_sharded<k>   ZeRO stage 2 / 3 with really sharded gradients / parameters (peer-memory kernels); every
                   step is split into two micro-steps so that the shard accumulation is exercised
  gpu_moe_a2a1     the same with the experts' rows exchanged through all_to_all_single (the measured baseline)
  gpu_moe_library1 / gpu_moe_fused   mixture-of-experts model, experts split over the ranks (peer-memory
                   dispatch / combine), dense parameters ZeRO-1 through library / fused communication
  gpu_cp64 / gpu_cp128   context-parallel attention (head size 64 / 128) against the single-GPU kernels on the full sequence
  cpu_fail_rank1   gloo; rank 1 raises before its first collective (failure-detection test)
environment: LLMK_TEST_LAYERS (dense model depth, default 2), LLMK_TEST_RECOMPUTE (default 0),
LLMK_TEST_GRAPH (replay the micro-step from CUDA graphs), LLMK_TEST_SKIP_STEP (index of a step whose optimizer update is left out, as the z-score guards of the trainer do)
Each rank writes ``rank<r>.pt`` with its per-step losses / norms and a parameter checksum sample.
"""
import datetime
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from llm_kittens_b200.models.config import ModelConfig  # noqa: E402
from llm_kittens_b200.parallel.comm import LibraryComm  # noqa: E402
from llm_kittens_b200.parallel.zero import ZeroPlan  # noqa: E402
from llm_kittens_b200.runtime.trainer import Trainer  # noqa: E402


def tiny_config():
    layers = int(os.environ.get("LLMK_TEST_LAYERS", "2"))
    return ModelConfig(family="gpt2", max_seq_len=64, vocab_size=512, padded_vocab_size=512, num_layers=layers, num_heads=2,
                       num_kv_heads=2, channels=128, hidden_dim=512)


def tiny_moe_config():
    # generous capacity: nothing is dropped, so the expert-parallel run equals a single process that
    # accumulates the ranks' micro-batches
    return ModelConfig(family="moe", max_seq_len=128, vocab_size=512, padded_vocab_size=512, num_layers=2, num_heads=2,
                       num_kv_heads=2, channels=128, hidden_dim=512, num_experts=8, top_k=2, capacity_factor=4.0,
                       aux_loss_coef=0.01)


def global_batches(cfg, steps, world, B, T):
    g = torch.Generator().manual_seed(1234)
    out = []
    for _ in range(steps):
        x = torch.randint(0, cfg.vocab_size, (world * B, T), generator=g, dtype=torch.int32)
        y = torch.randint(0, cfg.vocab_size, (world * B, T), generator=g, dtype=torch.int32)
        out.append((x, y))
    return out


def main():
    mode, out_dir = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cpu = mode.startswith("cpu")
    timeout = datetime.timedelta(seconds=int(os.environ.get("LLMK_TEST_PG_TIMEOUT", "120")))
    if cpu:
        dist.init_process_group("gloo", timeout=timeout)
        device = torch.device("cpu")
    else:
        torch.cuda.set_device(rank)
        device = torch.device("cuda", rank)
        dist.init_process_group("nccl", device_id=device, timeout=timeout)
    if mode == "cpu_fail_rank1":
        if rank == 1:
            raise RuntimeError("injected failure on rank 1 before its first collective")
        t = torch.ones(1)
        try:
            dist.all_reduce(t)  # the peer never joins: the short process-group timeout ends this with an error
            outcome = "completed"
        except Exception as e:  # noqa: BLE001
            outcome = "error:" + type(e).__name__
        torch.save({"outcome": outcome}, os.path.join(out_dir, f"rank{rank}.pt"))
        os._exit(0)
    if mode.startswith("gpu_cp"):
        # context-parallel attention: every rank holds one chunk of a seeded full sequence; rank 0 also runs the plain
        # single-GPU kernels on the whole sequence as the reference
        from llm_kittens_b200.ops import _native, attention
        from llm_kittens_b200.parallel.context import ContextParallelAttention

        HS = 128 if mode.endswith("128") else 64
        B, T, NH, NKVH = 2, 256, 4, 2
        W = (NH + 2 * NKVH) * HS
        g = torch.Generator().manual_seed(77)
        full = (torch.randn(B, world * T, W, generator=g) * 0.7).to(torch.bfloat16)
        dfull = (torch.randn(B, world * T, NH * HS, generator=g) * 0.5).to(torch.bfloat16)
        cp = ContextParallelAttention(B, T, NH, NKVH, HS, device, timeout_ms=60000)
        out = dqkv = None
        for _ in range(2):     # twice: the buffers are reused, and the results must be bit-identical
            prev = (out, dqkv)
            out = cp.forward(full[:, rank * T:(rank + 1) * T].contiguous().to(device)).clone()
            dqkv = cp.backward(dfull[:, rank * T:(rank + 1) * T].contiguous().to(device)).clone()
        torch.cuda.synchronize()
        _native.check_status()
        res = {"out": out.float().cpu(), "dqkv": dqkv.float().cpu(), "same": torch.equal(out, prev[0]) and torch.equal(dqkv, prev[1])}
        if rank == 0:
            fq = full.to(device)
            o, lse = attention.attention_fwd(fq, B, world * T, NH, NKVH, HS)
            d = attention.attention_bwd(dfull.to(device), fq, o, lse, B, world * T, NH, NKVH, HS)
            res["ref_out"], res["ref_dqkv"] = o.float().cpu(), d.float().cpu()
        torch.save(res, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
        return
    moe = "moe" in mode
    cfg = tiny_moe_config() if moe else tiny_config()
    B, T, steps = (2, 128, 3) if moe else (2, 64, 4)
    stage = int(mode[-1]) if mode[-1].isdigit() else 1
    if moe:
        from llm_kittens_b200.models.moe import MoETransformer
        from llm_kittens_b200.parallel.expert import LibraryExchange, PeerExchange

        # gpu_moe_a2a1: the baseline exchange through all_to_all_single
        exchange = LibraryExchange(device) if "a2a" in mode else PeerExchange(device, timeout_ms=60000)
        model = MoETransformer(cfg, device=device, recompute=0, exchange=exchange)
    elif cpu:
        from llm_kittens_b200.oracle.torch_model import TorchTransformer

        model = TorchTransformer(cfg, device=device, dtype=torch.float32)
    else:
        from llm_kittens_b200.models.transformer import Transformer

        model = Transformer(cfg, device=device, recompute=int(os.environ.get("LLMK_TEST_RECOMPUTE", "0")))
    model.init_weights(42)
    plan = ZeroPlan(cfg, world, rank, stage)
    if mode in ("gpu_fused", "gpu_fused0", "gpu_moe_fused"):
        from llm_kittens_b200.parallel.fused import FusedComm

        comm = FusedComm(plan, model, device, timeout_ms=60000)
    elif mode.startswith("gpu_sharded"):
        from llm_kittens_b200.parallel.sharded import ShardedComm

        comm = ShardedComm(plan, model, device, timeout_ms=60000)
    else:
        comm = LibraryComm(plan, None, device)
    trainer = Trainer(model, zero_stage=stage, use_master_weights=True, learning_rate=1e-3, weight_decay=0.1, comm=comm,
                      num_processes=world, rank=rank)
    if os.environ.get("LLMK_TEST_GRAPH"):
        trainer.enable_cuda_graph(True)   # step 0 runs eagerly, step 1 is captured, the later steps replay
    losses, norms = [], []
    leave = "leave" in mode
    if leave:
        # A rank leaves BETWEEN steps with none of its kernels or collectives in flight; the others learn of it at the
        # host-side step rendezvous, before they launch anything, and exit with the resume code.
        from llm_kittens_b200.runtime.watchdog import EXIT_RESUME, Watchdog, store_from_env

        def on_failure(msg):
            torch.save({"outcome": "peer_left", "message": msg, "losses": losses}, os.path.join(out_dir, f"rank{rank}.pt"))
            os._exit(EXIT_RESUME)

        wd = Watchdog(rank, world, deadline_s=3.0, store=store_from_env(rank, world), on_failure=on_failure)
    for step_index, (x, y) in enumerate(global_batches(cfg, steps, world, B, T)):
        if leave:
            if not cpu:
                torch.cuda.synchronize()
            if rank == 1 and step_index == 2:
                torch.save({"outcome": "left", "losses": losses}, os.path.join(out_dir, f"rank{rank}.pt"))
                os._exit(0)
            wd.enter_step(step_index)
        xs, ys = x[rank * B:(rank + 1) * B].contiguous(), y[rank * B:(rank + 1) * B].contiguous()
        if mode.startswith("gpu_sharded"):
            micro = [(xs[:1].contiguous(), ys[:1].contiguous()), (xs[1:].contiguous(), ys[1:].contiguous())]
        else:
            micro = [(xs, ys)]
        if step_index == int(os.environ.get("LLMK_TEST_SKIP_STEP", "-1")):
            from llm_kittens_b200.runtime.trainer import StepResult

            trainer.accumulate(micro)
            trainer.update(1e-3, skip=True)
            loss, norm, _ = trainer.read_scalars()
            trainer.skip_update()
            r = StepResult(loss=loss, grad_norm=norm, lr=1e-3, skipped=True)
        else:
            r = trainer.train_step(micro)
        losses.append(r.loss)
        norms.append(r.grad_norm)
    if not cpu:
        from llm_kittens_b200.ops import _native

        _native.check_status()
    torch.save({"losses": losses, "norms": norms, "params": (trainer.full_params() if not cpu else model.params).float().cpu()}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
