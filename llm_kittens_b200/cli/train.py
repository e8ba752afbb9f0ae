"""The training program behind ``train_gpt2cu`` and ``train_llama3cu``.

Flow (cf. the reference's main(), train_gpt2.cu:1737-2342): parse flags -> optional host-only dry run
(``-x 0``) -> process group -> model from checkpoint or descriptor -> data / eval loaders, tokenizer,
logger, LR schedule -> optional resume from the newest ``DONE_*`` checkpoint -> loop {validation,
HellaSwag-style eval, sampling, checkpointing, one optimizer step over ``grad_accum`` micro-batches,
z-score skip guards, step line}. Timing of a step is device time between CUDA events, reduced with
MAX over ranks; throughput is ``total_batch / step_time`` with the bias-corrected EMA(0.95) print-out.
"""
from __future__ import annotations

import os
import sys

import torch

from ..models.config import ModelConfig, config_from_descriptor
from ..parallel import zero as zero_mod
from ..utils import formats, nvtx
from ..utils.logger import Logger
from ..utils.outlier import NativeOutlierDetector as OutlierDetector
from ..utils.schedulers import LearningRateScheduler
from .flags import FlagError, TrainArgs, parse_flags


def printf0(rank: int, *a, **k) -> None:
    if rank == 0:
        print(*a, **k)
        sys.stdout.flush()


def load_config(source: str) -> tuple[ModelConfig, bool]:
    """(config, is_checkpoint) from a ``.bin`` path or a descriptor."""
    if source.endswith(".bin"):
        h = formats.read_header(source)
        cfg, fp32 = formats.config_from_model_header(h, source)
        expected = formats.HEADER_BYTES + cfg.num_parameters() * (4 if fp32 else 2)
        if os.path.getsize(source) != expected:
            raise formats.FormatError(f"{source}: payload size does not match the header")
        return cfg, True
    return config_from_descriptor(source), False


def dry_run(args: TrainArgs, trainer_name: str) -> int:
    """Host-only validation (``-x 0``): parses the model source, checks T, the ZeRO stage and that every
    tensor can be sharded over ``-pn`` processes. No CUDA call is made."""
    tag = "GPT" if trainer_name == "gpt2" else "Llama"
    if args.num_processes < 1:
        print(f"Invalid process count {args.num_processes} for {tag} dry run.", file=sys.stderr)
        return 1
    if not (0 <= args.process_rank < args.num_processes):
        print(f"Invalid process rank {args.process_rank} for {args.num_processes} processes in {tag} dry run.", file=sys.stderr)
        return 1
    if args.gpus_per_node < 1:
        print(f"Invalid GPUs-per-node count {args.gpus_per_node} for {tag} dry run.", file=sys.stderr)
        return 1
    try:
        zero_mod.validate_zero_stage(args.zero_stage)
        cfg, _ = load_config(args.load_filename)
    except (ValueError, OSError) as e:
        print(str(e), file=sys.stderr)
        return 1
    if args.T > cfg.max_seq_len:
        print(f"{tag} dry run sequence length T={args.T} exceeds model max_seq_len={cfg.max_seq_len}.", file=sys.stderr)
        return 1
    if trainer_name == "llama3" and (args.T % 16 != 0 or (args.B * args.T) % 128 != 0):
        print("Llama requires T % 16 == 0 and B*T % 128 == 0.", file=sys.stderr)
        return 1
    problems = zero_mod.validate_sharding(cfg, args.num_processes, args.zero_stage)
    if problems:
        for p in problems:
            print(f"ZeRO-{args.zero_stage} cannot shard {p}", file=sys.stderr)
        return 1
    n = cfg.num_parameters()
    print(f"{tag} dry run: source={args.load_filename}")
    print(f"{tag} dry run: max_seq_len={cfg.max_seq_len} vocab={cfg.vocab_size} padded_vocab={cfg.padded_vocab_size} "
          f"layers={cfg.num_layers} heads={cfg.num_heads} kv_heads={cfg.num_kv_heads} channels={cfg.channels}")
    print(f"{tag} dry run: parameters={n} bytes={2 * n}")
    print(f"{tag} dry run: ZeRO-{args.zero_stage} layout validated for {args.num_processes} process(es).")
    return 0


def run(argv: list[str], trainer_name: str) -> int:
    try:
        args = parse_flags(argv, trainer_name)
    except FlagError as e:
        print(str(e), file=sys.stderr)
        return 1
    if args.max_steps == 0:
        return dry_run(args, trainer_name)
    return train(args, trainer_name)


def resolve_processes(args: TrainArgs, env) -> tuple[int, int, str, int]:
    """(job size, this process's rank, rendezvous method, local device index) from the launcher's environment and the
    ``-p*`` flags: ``torch.distributed.run`` sets WORLD_SIZE / RANK / LOCAL_RANK; ``mpirun`` (how the reference's binaries
    are started, scripts/run_gpt2_124M.sh:45) sets OMPI_COMM_WORLD_*; otherwise ``-pn`` / ``-pr`` / ``-pg`` say it
    (one task per GPU under ``srun`` with ``-pi tcp`` or ``-pi fs``)."""
    env_world = int(env.get("WORLD_SIZE", "0"))
    local_default = None
    if env_world > 0 and args.nccl_init_method in ("mpi", "env"):
        world, rank, init = env_world, int(env.get("RANK", "0")), "env"
    elif args.nccl_init_method == "mpi" and "OMPI_COMM_WORLD_SIZE" in env:
        world, rank, init = int(env["OMPI_COMM_WORLD_SIZE"]), int(env["OMPI_COMM_WORLD_RANK"]), "mpi"
        local_default = env.get("OMPI_COMM_WORLD_LOCAL_RANK")
    else:
        world, rank, init = args.num_processes, args.process_rank, args.nccl_init_method
    if local_default is None:
        local_default = rank % max(1, args.gpus_per_node)
    return world, rank, init, int(env.get("LOCAL_RANK", local_default))


def train(args: TrainArgs, trainer_name: str) -> int:
    import torch.distributed as dist

    from ..models.transformer import Transformer
    from ..parallel.bootstrap import init_process_group, make_comm
    from ..runtime.checkpoint import load_checkpoint, save_checkpoint, prune_checkpoints
    from ..runtime.sampling import generate
    from ..runtime.trainer import Trainer
    from ..utils.dataloader import DataLoader, EvalLoader
    from ..utils.mfu import estimate_flops_per_token, flops_promised, gpu_utilization_info, mfu
    from ..utils.tokenizer import Tokenizer

    zero_mod.validate_zero_stage(args.zero_stage)
    # ---- processes
    world, rank, init, local = resolve_processes(args, os.environ)
    if world == 1 and int(os.environ.get("SLURM_NTASKS", "1") or 1) > 1 and int(os.environ.get("SLURM_PROCID", "0") or 0) == 0:
        print("warning: one of several slurm tasks, but no job size was given (-pn / -pr / -pi tcp|fs, or start the tasks "
              "through `python -m llm_kittens_b200.cli.recipes <name> --launcher slurm`): every task trains on its own",
              file=sys.stderr)
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        init_process_group(world, rank, init, args.server_ip, args.fs_path, device)

    B, T = args.B, args.T
    tokens_per_fwdbwd = B * T * world
    total_batch = args.total_batch_size if args.total_batch_size > 0 else tokens_per_fwdbwd
    if total_batch % tokens_per_fwdbwd != 0:
        printf0(rank, f"total batch size {total_batch} is not divisible by B*T*num_processes = {tokens_per_fwdbwd}")
        return 1
    grad_accum = total_batch // tokens_per_fwdbwd

    # ---- resume?
    resume_step = formats.find_max_step(args.output_log_dir) if args.resume == 1 else -1
    resuming = resume_step >= 0
    source = args.load_filename
    if resuming:
        source = formats.checkpoint_paths(args.output_log_dir, resume_step, rank)[0]
    cfg, is_ckpt = load_config(source)
    if cfg.family == "moe":
        from ..models.moe import MoETransformer as ModelCls
    else:
        ModelCls = Transformer
    if T > cfg.max_seq_len:
        printf0(rank, f"sequence length T={T} exceeds model max_seq_len={cfg.max_seq_len}")
        return 1
    model_kw = {}
    if cfg.family == "moe" and world > 1:
        # the experts are split over the ranks (the ZeRO plan gives every expert one owner): rows travel through the
        # peer-memory exchange inside one NVLink domain, through all_to_all_single otherwise
        from ..parallel.expert import LibraryExchange, PeerExchange

        if cfg.num_experts % world != 0:
            printf0(rank, f"{cfg.num_experts} experts cannot be split over {world} processes")
            return 1
        try:
            model_kw["exchange"] = PeerExchange(device)
        except Exception as e:      # no peer memory between the ranks (several nodes, more than 8 ranks)
            printf0(rank, f"[llm_kittens_b200] peer-memory expert exchange unavailable ({e}); using all_to_all_single")
            model_kw["exchange"] = LibraryExchange(device)
    model = ModelCls(cfg, device=device, recompute=args.recompute, **model_kw)
    if is_ckpt:
        _, flat = formats.read_model(source, device="cpu")
        model.load_parameters(flat.to(device))
    else:
        model.init_weights(42)
    model.allocate(B, T)
    plan = zero_mod.ZeroPlan(cfg, world, rank, args.zero_stage)
    comm = make_comm(plan, model, world, rank, device)
    trainer = Trainer(model, zero_stage=args.zero_stage, use_master_weights=bool(args.use_master_weights),
                      learning_rate=args.learning_rate, weight_decay=args.weight_decay, comm=comm, num_processes=world, rank=rank)
    # micro-steps replayed from CUDA graphs where the model and the communication path can be captured (dense models,
    # one process or the fused ZeRO-0/1 path); the first step runs eagerly, the second one is captured
    if os.environ.get("LLMK_CUDA_GRAPH", "1") != "0":
        trainer.enable_cuda_graph(True)

    # ---- config table
    printf0(rank, "+-----------------------+----------------------------------------------------+")
    for k, v in (("train data pattern", args.train_data_pattern), ("val data pattern", args.val_data_pattern),
                 ("output log dir", args.output_log_dir), ("checkpoint_every", args.checkpoint_every), ("resume", args.resume),
                 ("micro batch size B", B), ("sequence length T", T), ("total batch size", total_batch),
                 ("LR scheduler", args.lr_scheduler_type), ("learning rate (LR)", args.learning_rate),
                 ("warmup iterations", args.warmup_iterations), ("final LR fraction", args.final_learning_rate_frac),
                 ("weight decay", args.weight_decay), ("max_steps", args.max_steps), ("use_master_weights", args.use_master_weights),
                 ("recompute", args.recompute), ("device", torch.cuda.get_device_name(local)), ("precision", "BF16"),
                 ("load_filename", args.load_filename), ("max_sequence_length T", cfg.max_seq_len),
                 ("vocab_size V", cfg.vocab_size), ("padded_vocab_size Vp", cfg.padded_vocab_size),
                 ("num_layers L", cfg.num_layers), ("num_heads NH", cfg.num_heads), ("channels C", cfg.channels),
                 ("num_parameters", cfg.num_parameters()), ("num_processes", world), ("zero_stage", args.zero_stage),
                 ("communication", type(comm).__name__ + (f" + {type(model_kw['exchange']).__name__}" if model_kw else "")),
                 ("grad_accum_steps", grad_accum)):
        printf0(rank, f"| {k:<21} | {str(v):<50} |")
    printf0(rank, "+-----------------------+----------------------------------------------------+")

    # ---- data
    train_loader = DataLoader(args.train_data_pattern, B, T, rank, world, should_shuffle=True, ring=grad_accum + 1)
    val_loader = DataLoader(args.val_data_pattern, B, T, rank, world, should_shuffle=False)
    train_num_batches = train_loader.num_tokens // total_batch
    if args.max_steps > 0:
        train_num_batches = args.max_steps
    val_num_batches = max(1, min(args.val_max_steps, val_loader.num_tokens // tokens_per_fwdbwd))
    eval_loader = None
    hs_path = "dev/data/hellaswag/hellaswag_val.bin"
    if args.hellaswag_eval and os.path.exists(hs_path) and B >= 4:
        eval_loader = EvalLoader(hs_path, B, T, rank, world)
    tok_path = "gpt2_tokenizer.bin" if cfg.family != "llama3" else "llama3_tokenizer.bin"
    tokenizer = Tokenizer(tok_path) if os.path.exists(tok_path) else None
    logger = Logger(args.output_log_dir, rank, resume=resuming)
    sched = LearningRateScheduler(args.lr_scheduler_type, args.learning_rate, args.warmup_iterations, train_num_batches,
                                  args.final_learning_rate_frac)

    # host watchdog (LLMK_WATCHDOG_SECONDS > 0): a step that takes longer than the deadline, or a peer whose heartbeat
    # stops, ends this process with the exit code that the supervisor maps to "resume from the last checkpoint"
    watchdog = None
    rendezvous = os.environ.get("LLMK_WATCHDOG_RENDEZVOUS", "0") not in ("", "0")   # host-side meeting point before every step
    deadline = float(os.environ.get("LLMK_WATCHDOG_SECONDS", "0") or 0)
    if deadline > 0:
        from ..runtime.watchdog import Watchdog, store_from_env
        store = None
        if world > 1:
            if args.server_ip:      # -pi tcp / mpi over several nodes: the heartbeat store lives beside rank 0 as well
                os.environ.setdefault("MASTER_ADDR", args.server_ip)
            # every rank must come to the same decision, or rank 0 would wait for heartbeats that nobody can send
            if "MASTER_ADDR" in os.environ or world <= args.gpus_per_node:
                store = store_from_env(rank, world)
            else:                   # e.g. -pi fs over several nodes: no address of rank 0 is known
                printf0(rank, "[llm_kittens_b200] no address for the heartbeat store (set MASTER_ADDR or -ps): the watchdog "
                              "watches the step deadline only")
        watchdog = Watchdog(rank, world, deadline, store=store)
        watchdog.start()

    can_sample = not model_kw
    if not can_sample and args.sample_every > 0:
        printf0(rank, "sampling (-s) is switched off: with the experts split over the ranks a forward pass needs all of them")
    step = 0
    if resuming:
        step = load_checkpoint(args.output_log_dir, resume_step, trainer, train_loader, world, rank)
        printf0(rank, f"resumed from step {step}")

    # ---- loop
    peak = flops_promised(torch.cuda.get_device_name(local), "bf16")
    embed_params = 0 if cfg.family == "llama3" else cfg.max_seq_len * cfg.channels
    flops_tok = estimate_flops_per_token(cfg.num_parameters(), cfg.num_layers, cfg.channels, T, embed_params)
    loss_det, norm_det = OutlierDetector(), OutlierDetector()
    ema_tps = 0.0
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total_ms, timed_steps = 0.0, 0
    losses_host = torch.empty(B * T, dtype=torch.float32).pin_memory()
    nvtx.profiler_start()   # with LLMK_NVTX=1: the capture range of a profiler ends after the third step, as in the reference
    first_loop_step = step
    while step <= train_num_batches:
        last_step = step == train_num_batches
        if watchdog is not None:
            watchdog.beat(step)
            if rendezvous:
                # nothing of this rank is in flight here: a peer that left or hangs is noticed before the next launch
                torch.cuda.synchronize()
                watchdog.enter_step(step)
        # validation
        if step % max(1, args.val_loss_every) == 0 or last_step:
            val_loader.reset()
            acc = torch.zeros(1, device=device)
            with nvtx.nvtx_range("validation"):
                for _ in range(val_num_batches):
                    x, y = val_loader.next_batch()
                    model.forward(x, y, compute_dlogits=False)
                    acc += model.acts["loss_acc"]
            acc /= val_num_batches
            comm.all_reduce_scalar(acc, "avg")
            val_loss = float(acc.item())
            printf0(rank, f"val loss {val_loss:f}")
            logger.log_val(step, val_loss)
        # multiple-choice eval
        if eval_loader is not None and (step % max(1, args.val_loss_every) == 0 or last_step):
            eval_loader.reset()
            correct = torch.zeros(1, device=device)
            for _ in range(eval_loader.num_batches):
                x, y = eval_loader.next_batch()
                model.forward(x, y, compute_dlogits=False)
                losses_host.copy_(model.acts["losses"], non_blocking=False)
                correct += eval_loader.stat_losses(losses_host.numpy())
            comm.all_reduce_scalar(correct, "sum")
            accy = float(correct.item()) / eval_loader.num_examples
            printf0(rank, f"HellaSwag: {int(correct.item())}/{eval_loader.num_examples} = {accy:f}")
            logger.log_eval(step, accy)
        # sampling (one process; an expert-parallel forward needs every rank, so those runs do not sample)
        if rank == 0 and can_sample and args.sample_every > 0 and step > 0 and (step % args.sample_every == 0 or last_step):
            eot = tokenizer.eot_token if tokenizer else 50256 if cfg.family != "llama3" else 128001
            toks = generate(model, [eot], args.genT, rng_state=1337)
            if tokenizer is not None:
                text = "".join(Tokenizer.safe_text(tokenizer.decode(t)) for t in toks[1:])
                print("generating:\n---\n" + text + "\n---")
            else:
                print("generating:\n---\n" + " ".join(str(t) for t in toks[1:]) + "\n---")
        # checkpoint
        if args.checkpoint_every > 0 and args.output_log_dir and ((step > 0 and step % args.checkpoint_every == 0) or last_step) \
                and not (resuming and step == resume_step):
            with nvtx.nvtx_range("checkpoint"):
                save_checkpoint(args.output_log_dir, step, trainer, train_loader, world, rank, comm)
            prune_checkpoints(args.output_log_dir, step, args.checkpoint_every, args.checkpoints_keep, args.major_checkpoint_every,
                              world, rank)
        if last_step:
            break

        if step == first_loop_step + 3:
            nvtx.profiler_stop()
        ev0.record()
        if args.overfit_single_batch and step > 0:
            batches = [(train_loader.inputs, train_loader.targets)] * grad_accum
            trainer.accumulate(batches)
        else:
            trainer.begin_step()
            for micro in range(grad_accum):
                x, y = train_loader.next_batch()
                trainer.micro_step(x, y, micro, grad_accum)
        lr = sched.get(step)
        guards = args.skip_update_lossz != 0.0 or args.skip_update_gradz != 0.0
        if guards:
            trainer.update(lr, skip=True)   # reduction, loss, norm and clip coefficient only
            loss, norm, bad = trainer.read_scalars()
            zloss, zgrad = loss_det.update(loss), norm_det.update(norm)
            skip = bad or (args.skip_update_lossz != 0.0 and zloss == zloss and zloss > args.skip_update_lossz) or \
                (args.skip_update_gradz != 0.0 and zgrad == zgrad and zgrad > args.skip_update_gradz)
            if skip:
                printf0(rank, f"skipping update: loss z-score {zloss:.2f}, grad-norm z-score {zgrad:.2f}")
                trainer.skip_update()
            else:
                trainer.apply_update(lr)
        else:
            trainer.update(lr)
            loss, norm, bad = trainer.read_scalars()
            zloss, zgrad = loss_det.update(loss), norm_det.update(norm)
        ev1.record()
        ev1.synchronize()
        ms = torch.tensor([ev0.elapsed_time(ev1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        ms = float(ms.item())
        step += 1
        tps = total_batch / (ms / 1e3)
        if step > 1:
            total_ms += ms
            timed_steps += 1
            ema_tps = 0.95 * ema_tps + 0.05 * tps
            bias_corrected = ema_tps / (1.0 - 0.95 ** timed_steps)
        else:
            bias_corrected = tps
        m = mfu(bias_corrected, flops_tok, peak) if peak > 0 else -1.0
        printf0(rank, "step %4d/%d | loss %7.6f (%+.2fz)| norm %6.4f (%+.2fz)| lr %.2e | %.2f ms | %.1f%% bf16 MFU | %.0f tok/s"
                % (step, train_num_batches, loss, zloss, norm, zgrad, lr, ms, 100 * m, bias_corrected))
        if args.log_gpu_every > 0 and step % args.log_gpu_every == 0 and rank == 0:
            info = gpu_utilization_info(local)
            if info:
                print("                  compute %d%% | memory: %d%% | clock %d/%d MHz | power %.0f/%.0f W | temp %d C | throttle 0x%x"
                      % (info["gpu_util"], info["mem_util"], info["clock_mhz"], info["max_clock_mhz"], info["power_w"],
                         info["power_limit_w"], info["temperature_c"], info["throttle_reasons"]))
        logger.log_train(step - 1, loss, lr, norm)
    if watchdog is not None:
        watchdog.stop()
    if timed_steps:
        printf0(rank, f"total average iteration time: {total_ms / timed_steps:f} ms")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0
