"""Launch recipes: the hyper-parameter presets of the reference's launch scripts as one table and one command.

    python -m llm_kittens_b200.cli.recipes list
    python -m llm_kittens_b200.cli.recipes gpt2_124M --gpus 8 [--out DIR] [--max-steps N] [--train "PATTERN"] [--val "PATTERN"]
    python -m llm_kittens_b200.cli.recipes llama3_8B --launcher slurm --rendezvous fs --fs-path /shared/run1     # one task per GPU under srun
    python -m llm_kittens_b200.cli.recipes gpt2_124M_2nodes --launcher mpi                                          # one task per GPU under mpirun
    python -m llm_kittens_b200.cli.recipes gpt2_350M --dry-run -- -z 2 -r 1                                          # print the command; extra trainer flags after --

Each preset carries the trainer flags of one script of the reference (scripts/run_gpt2_124M.sh:44-63,
run_gpt2_350M.sh:27-44, run_gpt2_774M.sh:27-44, run_gpt2_1558M.sh:25-43, run_gpt3_125M.sh:25-46, run_llama3_1B.sh:45-66,
multi_node/run_gpt2_124M_{mpi,tcp,fs}.*, multi_node/run_llama3_8B_fs.sbatch:77-104), so a run started here trains with
the same batch, schedule, evaluation and checkpoint settings. What differs is the plumbing around them:

* ``--launcher torchrun`` (default): this command starts ``torch.distributed.run`` with one process per GPU on this node
  (``--nnodes`` / ``--node-rank`` / ``--master-addr`` for more nodes) inside the restart loop of ``cli/supervise.py``,
  which replaces the scripts' ``while true; do ...; sleep 1; done`` (the trainer gets ``-y 1`` from the second attempt on).
* ``--launcher slurm`` / ``--launcher mpi``: this command IS one task of an ``srun`` / ``mpirun`` job (one task per GPU).
  It reads its rank and the job size from the scheduler's environment and runs the trainer in this process with the
  ``-pn / -pr / -pg / -pi / -ps / -pf`` rendezvous flags of the reference (tcp: rank 0 listens on ``--server-ip``; fs: a
  file under ``--fs-path``; mpi: Open MPI's environment). No binary is copied to the other hosts: the package is
  expected on a shared path or installed on every node.
"""
from __future__ import annotations

import argparse
import os
import shlex
import sys
from dataclasses import dataclass

from . import flags as flags_mod
from . import supervise as supervise_mod


@dataclass(frozen=True)
class Recipe:
    trainer: str                      # "gpt2" | "llama3": which trainer module runs it
    model: str                        # -e descriptor
    out_dir: str                      # default -o
    max_steps: int                    # default -x
    train: str                        # default -i pattern
    val: str                          # default -j pattern
    flags: tuple                      # the remaining trainer flags, in the order of the reference's script
    nodes: int = 1                    # how many 8-GPU nodes the preset's total batch was chosen for
    note: str = ""


def _f(text: str) -> tuple:
    return tuple(text.split())


_FW10 = ("dev/data/fineweb10B/fineweb_train_*.bin", "dev/data/fineweb10B/fineweb_val_*.bin")
_FW100 = ("dev/data/fineweb100B/fineweb_train_*.bin", "dev/data/fineweb100B/fineweb_val_*.bin")
_EDU100 = ("dev/data/edu_fineweb100B/edu_fineweb_train_*.bin", "dev/data/edu_fineweb100B/edu_fineweb_val_*.bin")

RECIPES: dict[str, Recipe] = {
    "gpt2_124M": Recipe("gpt2", "d12", "log_gpt2_124M", 18865, *_FW10,
                        _f("-v 250 -s 20000 -g 144 -h 1 -b 64 -t 1024 -d 524288 -r 0 -z 1 -c 0.1 -l 0.0006 -q 0.0 -u 700 -n 5000"),
                        note="the headline configuration: 10B FineWeb tokens, 524288 tokens per step"),
    "gpt2_350M": Recipe("gpt2", "d24", "log_gpt2_350M", 60000, *_FW100,
                        _f("-v 250 -s 100000 -g 144 -h 1 -b 64 -t 1024 -d 524288 -r 0 -z 1 -c 0.1 -l 0.0003 -q 0.0 -u 700 -n 2000 -ge 1")),
    "gpt2_774M": Recipe("gpt2", "d36", "log_gpt2_774M", 286102, *_FW100,
                        _f("-v 250 -s 300000 -g 144 -h 1 -b 32 -t 1024 -d 524288 -r 0 -z 1 -c 0.1 -l 0.00025 -q 0.0 -u 700 -n 4000 -ge 1")),
    "gpt2_1558M": Recipe("gpt2", "d48", "log_gpt2_1558M", 32000, *_EDU100,
                         _f("-v 250 -s 300000 -g 384 -h 1 -b 16 -t 1024 -d 1048576 -r 0 -z 1 -c 0.1 -k cosine -l 0.0006 -q 0.1 -u 700 "
                            "-n 2000 -ge 1")),
    "gpt3_125M": Recipe("gpt2", "gpt3:c768", "log_gpt3_125M", 572204, *_FW100,
                        _f("-v 250 -s 20000 -g 144 -h 1 -b 32 -t 2048 -d 524288 -r 0 -z 1 -c 0.1 -l 0.0006 -q 0.1 -u 700 -n 10000 -nk 5 "
                           "-nm 50000 -ge 1 -sl 7.0 -sg 7.0")),
    "llama3_1B": Recipe("llama3", "llama3:1B", "log_llama3_1B", 57220, *_EDU100,
                        _f("-v 250 -m 20 -s 20000 -g 144 -h 1 -b 32 -t 2048 -d 524288 -r 0 -z 1 -c 0.1 -l 0.0003 -q 0.1 -u 2000 -n 5000 "
                           "-nk 5 -nm 50000 -sl 7.0 -sg 7.0")),
    # two 8-GPU nodes, total batch 2M tokens (multi_node/run_gpt2_124M_{tcp,fs}.sbatch; the mpi script differs in -q / -n)
    "gpt2_124M_2nodes": Recipe("gpt2", "d12", "log_gpt2_124M_multi", 18865, *_FW10,
                               _f("-v 250 -s 20000 -g 144 -h 1 -b 64 -t 1024 -d 2097152 -r 0 -z 1 -c 0.1 -l 0.0006 -q 0.0 -u 700 -n 5000"),
                               nodes=2),
    # sharded gradients and recomputed activations (multi_node/run_llama3_8B_fs.sbatch: B=4, T=2048, ZeRO-2, -r 1)
    "llama3_8B": Recipe("llama3", "llama3:8B", "log_llama3_8B_multi", 57220, *_FW100,
                        _f("-v 250 -m 20 -s 20000 -g 144 -h 1 -b 4 -t 2048 -d 524288 -r 1 -z 2 -c 0.1 -l 0.0003 -q 0.1 -u 2000 -n 5000 "
                           "-nk 5 -nm 50000 -sl 7.0 -sg 7.0"),
                        nodes=2, note="a B200 holds the 8B model with ZeRO-3 on one node: add `-- -z 3 -b 1 -t 4096` for that layout"),
}

TRAINER_MODULES = {"gpt2": "llm_kittens_b200.cli.train_gpt2cu", "llama3": "llm_kittens_b200.cli.train_llama3cu"}


def trainer_flags(r: Recipe, out_dir: str | None = None, max_steps: int | None = None, train: str | None = None,
                  val: str | None = None, extra: list[str] | None = None) -> list[str]:
    """The trainer's flag list for a preset; ``extra`` flags come last and therefore win over the preset's."""
    argv = ["-i", train or r.train, "-j", val or r.val, "-o", out_dir or r.out_dir, *r.flags,
            "-x", str(max_steps if max_steps is not None else r.max_steps), "-e", r.model]
    argv += list(extra or [])
    flags_mod.parse_flags(argv, r.trainer)       # a preset that the parser would refuse is a bug here, not at launch time
    return argv


def torchrun_command(r: Recipe, tflags: list[str], gpus: int, nnodes: int = 1, node_rank: int = 0, master_addr: str = "127.0.0.1",
                     master_port: int = 29500) -> list[str]:
    return [sys.executable, "-m", "torch.distributed.run", f"--nnodes={nnodes}", f"--node-rank={node_rank}",
            f"--nproc-per-node={gpus}", "--master-addr", master_addr, "--master-port", str(master_port),
            "-m", TRAINER_MODULES[r.trainer], *tflags]


def scheduler_rank(launcher: str, env=os.environ) -> tuple[int, int, int]:
    """(job size, this task's rank, tasks per node) from the scheduler's environment."""
    need = {"slurm": ("SLURM_NTASKS", "SLURM_PROCID"), "mpi": ("OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_RANK")}.get(launcher, ())
    missing = [k for k in need if k not in env]
    if missing:
        raise ValueError(f"--launcher {launcher} must run as a task of that scheduler's job: {', '.join(missing)} not set")
    if launcher == "slurm":
        n, rank = int(env["SLURM_NTASKS"]), int(env["SLURM_PROCID"])
        per_node = env.get("SLURM_NTASKS_PER_NODE", "8").split("(")[0]
        return n, rank, int(per_node)
    if launcher == "mpi":
        n, rank = int(env["OMPI_COMM_WORLD_SIZE"]), int(env["OMPI_COMM_WORLD_RANK"])
        return n, rank, int(env.get("OMPI_COMM_WORLD_LOCAL_SIZE", "8"))
    raise ValueError(f"unknown launcher {launcher}")


def rendezvous_flags(launcher: str, rendezvous: str, server_ip: str = "", fs_path: str = "", env=os.environ) -> list[str]:
    """``-pn/-pr/-pg/-pi/-ps/-pf`` for one task of an srun / mpirun job (train_gpt2.cu:1650-1668 for their meaning)."""
    n, rank, per_node = scheduler_rank(launcher, env)
    out = ["-pn", str(n), "-pr", str(rank), "-pg", str(per_node), "-pi", rendezvous]
    if rendezvous == "tcp":
        if not server_ip:
            raise ValueError("--rendezvous tcp needs --server-ip (the address of the node that runs rank 0)")
        out += ["-ps", server_ip]
    elif rendezvous == "fs":
        if not fs_path:
            raise ValueError("--rendezvous fs needs --fs-path (a directory that every node sees)")
        out += ["-pf", fs_path]
    elif rendezvous == "mpi":
        if server_ip:      # more than one node: where rank 0 listens (else MASTER_ADDR, else this host)
            out += ["-ps", server_ip]
    else:
        raise ValueError(f"unknown rendezvous {rendezvous}")
    return out


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    extra: list[str] = []
    if "--" in argv:
        cut = argv.index("--")
        argv, extra = argv[:cut], argv[cut + 1:]
    ap = argparse.ArgumentParser(prog="llm_kittens_b200.cli.recipes", description=__doc__.split("\n\n")[0])
    ap.add_argument("recipe", help="a preset name, or `list`")
    ap.add_argument("--gpus", type=int, default=8, help="processes (GPUs) on this node [torchrun launcher]")
    ap.add_argument("--nnodes", type=int, default=1)
    ap.add_argument("--node-rank", type=int, default=0)
    ap.add_argument("--master-addr", default="127.0.0.1")
    ap.add_argument("--master-port", type=int, default=29500)
    ap.add_argument("--launcher", choices=("torchrun", "slurm", "mpi"), default="torchrun")
    ap.add_argument("--rendezvous", choices=("tcp", "fs", "mpi"), default=None, help="slurm / mpi launchers: the trainer's -pi")
    ap.add_argument("--server-ip", default="")
    ap.add_argument("--fs-path", default="")
    ap.add_argument("--out", default=None)
    ap.add_argument("--max-steps", type=int, default=None)
    ap.add_argument("--train", default=None)
    ap.add_argument("--val", default=None)
    ap.add_argument("--max-restarts", type=int, default=20)
    ap.add_argument("--dry-run", action="store_true", help="print the command instead of running it")
    args = ap.parse_args(argv)

    if args.recipe == "list":
        for name, r in RECIPES.items():
            fl = flags_mod.parse_flags(trainer_flags(r), r.trainer)
            print(f"{name:18s} {r.model:10s} B={fl.B} T={fl.T} tokens/step={fl.total_batch_size} zero={fl.zero_stage} recompute={fl.recompute} "
                  f"lr={fl.learning_rate:g} steps={r.max_steps} nodes={r.nodes}" + (f"  ({r.note})" if r.note else ""))
        return 0
    if args.recipe not in RECIPES:
        print(f"unknown recipe {args.recipe}; known: {', '.join(RECIPES)}", file=sys.stderr)
        return 2
    r = RECIPES[args.recipe]
    try:
        if args.launcher == "torchrun":
            tflags = trainer_flags(r, args.out, args.max_steps, args.train, args.val, extra)
            cmd = torchrun_command(r, tflags, args.gpus, args.nnodes, args.node_rank, args.master_addr, args.master_port)
        else:
            rdv = rendezvous_flags(args.launcher, args.rendezvous or ("mpi" if args.launcher == "mpi" else "tcp"), args.server_ip,
                                   args.fs_path)
            tflags = trainer_flags(r, args.out, args.max_steps, args.train, args.val, rdv + extra)
            cmd = [sys.executable, "-m", TRAINER_MODULES[r.trainer], *tflags]
    except (ValueError, flags_mod.FlagError) as e:
        print(f"recipes: {e}", file=sys.stderr)
        return 2
    parsed = flags_mod.parse_flags(tflags, r.trainer)
    if args.dry_run:
        print(" ".join(shlex.quote(c) for c in cmd))
        return 0
    if args.launcher == "torchrun":
        return supervise_mod.supervise(cmd, parsed.output_log_dir, parsed.max_steps, args.max_restarts)
    # one task of a scheduler's job: the scheduler owns restarts; run the trainer in this process
    from . import train as train_mod

    return int(train_mod.run(tflags, r.trainer) or 0)


if __name__ == "__main__":
    sys.exit(main())
