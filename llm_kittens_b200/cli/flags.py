"""Command-line flag parser of the trainers: ``-x value`` pairs with one- or two-letter names, the
same letters, defaults and meanings as the reference binaries (train_gpt2.cu:1618-1668, 1739-1820;
train_llama3.cu:1354-1461). Unknown flags and malformed pairs raise ``FlagError`` with the usage text.
"""
from __future__ import annotations

from dataclasses import dataclass, field


class FlagError(ValueError):
    pass


@dataclass
class TrainArgs:
    train_data_pattern: str = "dev/data/tinyshakespeare/tiny_shakespeare_train.bin"   # -i
    val_data_pattern: str = "dev/data/tinyshakespeare/tiny_shakespeare_val.bin"       # -j
    load_filename: str = "gpt2_124M_bf16.bin"                                         # -e
    output_log_dir: str | None = None                                                 # -o
    checkpoint_every: int = 0                                                         # -n
    checkpoints_keep: int = 0                                                         # -nk
    major_checkpoint_every: int = 0                                                   # -nm
    resume: int = 0                                                                   # -y
    B: int = 4                                                                        # -b
    T: int = 1024                                                                     # -t
    total_batch_size: int = -1                                                        # -d
    max_steps: int = -1                                                               # -x
    lr_scheduler_type: str = "cosine"                                                 # -k
    learning_rate: float = 3e-4                                                       # -l
    warmup_iterations: int = 0                                                        # -u
    final_learning_rate_frac: float = 1.0                                             # -q
    weight_decay: float = 0.0                                                         # -c
    skip_update_lossz: float = 0.0                                                    # -sl
    skip_update_gradz: float = 0.0                                                    # -sg
    val_loss_every: int = 20                                                          # -v
    val_max_steps: int = 20                                                           # -m
    sample_every: int = 20                                                            # -s
    genT: int = 64                                                                    # -g
    hellaswag_eval: int = 0                                                           # -h
    overfit_single_batch: int = 0                                                     # -a
    override_enable_tf32: int = 1                                                     # -f
    use_master_weights: int = 1                                                       # -w
    gelu_fusion: int = 1                                                              # -ge
    recompute: int = 1                                                                # -r
    zero_stage: int = 0                                                               # -z
    log_gpu_every: int = -1                                                           # -lg
    num_processes: int = 1                                                            # -pn
    process_rank: int = 0                                                             # -pr
    gpus_per_node: int = 8                                                            # -pg
    nccl_init_method: str = "mpi"                                                     # -pi
    fs_path: str = ""                                                                 # -pf
    server_ip: str = ""                                                               # -ps
    extras: dict = field(default_factory=dict)


# flag -> (field, type)
_GPT_FLAGS = {
    "i": ("train_data_pattern", str), "j": ("val_data_pattern", str), "e": ("load_filename", str),
    "o": ("output_log_dir", str), "n": ("checkpoint_every", int), "nk": ("checkpoints_keep", int),
    "nm": ("major_checkpoint_every", int), "y": ("resume", int), "b": ("B", int), "t": ("T", int),
    "d": ("total_batch_size", int), "x": ("max_steps", int), "k": ("lr_scheduler_type", str),
    "l": ("learning_rate", float), "u": ("warmup_iterations", int), "q": ("final_learning_rate_frac", float),
    "c": ("weight_decay", float), "sl": ("skip_update_lossz", float), "sg": ("skip_update_gradz", float),
    "v": ("val_loss_every", int), "m": ("val_max_steps", int), "s": ("sample_every", int), "g": ("genT", int),
    "h": ("hellaswag_eval", int), "a": ("overfit_single_batch", int), "f": ("override_enable_tf32", int),
    "w": ("use_master_weights", int), "ge": ("gelu_fusion", int), "r": ("recompute", int), "z": ("zero_stage", int),
    "lg": ("log_gpu_every", int), "pn": ("num_processes", int), "pr": ("process_rank", int),
    "pg": ("gpus_per_node", int), "pi": ("nccl_init_method", str), "pf": ("fs_path", str), "ps": ("server_ip", str),
}
# the Llama trainer has no -ge -f -a -lg -w
_LLAMA_FLAGS = {k: v for k, v in _GPT_FLAGS.items() if k not in ("ge", "f", "a", "lg", "w")}

USAGE_GPT = """Usage:   train_gpt2cu [options]
Options:
  -i <string> train data filename pattern          -j <string> val data filename pattern
  -e <string> input .bin checkpoint or descriptor dN | gpt2:dN | gpt3:cN | moe:dN
  -o <string> output log dir (default = none)      -lg <int>   log gpu info every x steps (default = -1; disabled)
  -n <int>    write checkpoints every how many steps?   -nk <int> keep last k   -nm <int> every how many steps is major?
  -y <int>    resume optimization found inside output log dir? (0=restart/overwrite, 1=resume)
  -b <int>    (per-GPU, micro) batch size B (default = 4)     -t <int> sequence length T (default = 1024)
  -d <int>    total desired batch size (default = B * T * num_processes, i.e. no grad accumulation)
  -x <int>    max_steps of optimization to run (-1 (default) = one epoch; 0 = host-only dry run)
  -k <string> learning rate scheduler: cosine | linear | constant | wsd (default = cosine)
  -l <float>  learning rate (default = 3e-4f)      -u <int> learning rate warmup iterations (default = 0)
  -q <float>  learning rate decay: final fraction, at end of training (default = 1.0 (no decay))
  -c <float>  weight decay (default = 0.0f)
  -sl <float> outlier stability: skip update if loss goes above this in zscore (0.0f=off)
  -sg <float> outlier stability: skip update if grad_norm goes above this in zscore (0.0f=off)
  -v <int>    val_loss_every   -m <int> val_max_steps   -s <int> sample_every   -g <int> genT   -h <int> hellaswag_eval
  -a <int>    overfit a single batch? 0/1        -f <int> enable_tf32 override (no effect)
  -w <int>    keep f32 copy of weights for the optimizer? (default: 1)
  -ge <int>   gelu fusion (kept for compatibility; the GEMM epilogue is always fused)
  -z <int>    zero_stage 0..3                    -r <int> recompute: 0 none, 1 GELU, 2 GELU+norms, 3 whole blocks
  -pn <int>   num_processes   -pr <int> process_rank   -pg <int> gpus_per_node
  -pi <string> init method: mpi | tcp | fs | env   -pf <string> fs_path   -ps <string> server_ip
"""
USAGE_LLAMA = USAGE_GPT.replace("train_gpt2cu", "train_llama3cu").replace(
    "descriptor dN | gpt2:dN | gpt3:cN | moe:dN", "descriptor llama3:1B | llama3:8B | llama3.1:8B | llama3.2:1B")


def parse_flags(argv: list[str], trainer: str = "gpt2") -> TrainArgs:
    """``argv``: the arguments after the program name."""
    table = _GPT_FLAGS if trainer == "gpt2" else _LLAMA_FLAGS
    usage = USAGE_GPT if trainer == "gpt2" else USAGE_LLAMA
    args = TrainArgs()
    if trainer == "llama3":
        args.load_filename = "llama3:1B"
        args.T = 2048
        args.max_steps = 0
        args.recompute = 0
    if len(argv) % 2 != 0:
        raise FlagError("every flag needs a value\n" + usage)
    for i in range(0, len(argv), 2):
        flag, val = argv[i], argv[i + 1]
        if not flag.startswith("-") or not (2 <= len(flag) <= 3):
            raise FlagError(f"bad flag {flag!r}\n" + usage)
        key = flag[1:]
        if key not in table:
            raise FlagError(f"unknown flag {flag!r}\n" + usage)
        name, typ = table[key]
        try:
            setattr(args, name, typ(val))
        except ValueError:
            raise FlagError(f"flag {flag} expects a value of type {typ.__name__}, got {val!r}\n" + usage) from None
    return args
