"""Run-validation commands: ``python -m llm_kittens_b200.cli.check <command> …``.

* ``log MAIN_LOG [--final-step N] [--max-train-loss X] [--max-val-loss X] [--no-decrease]`` — the threshold /
  decrease checks of the reference's ``dev/validate_training_log.py`` (1-179) on a ``main.log``.
* ``compare LOG_A LOG_B [--rel-tol R] [--abs-tol A]`` — curve comparison of two runs, as in
  ``dev/compare_training_logs.py`` (1-125): how "N GPUs == 1 GPU" is checked.
* ``zero-layout [--models …] [--world …]`` — recomputes the ZeRO shard intervals of every model descriptor at every
  world size and checks that they tile each tensor exactly (``dev/validate_zero_layout.py:1-174``).
* ``checkpoint DIR [--step N]`` — header / size / DONE-marker checks of a checkpoint directory
  (``dev/validate_llama_checkpoint_artifacts.py``).

Every command prints its findings and exits 1 if there are any.
"""
from __future__ import annotations

import argparse
import os
import sys

from ..models.config import config_from_descriptor
from ..parallel import zero
from ..utils import formats
from ..utils.logger import compare_logs, validate_log

DEFAULT_MODELS = ["d12", "d24", "d36", "d48", "gpt3:c768", "gpt3:c1024", "gpt3:c2048", "gpt3:c4096", "gpt3:c12288",
                  "llama3.2:1B", "llama3:8B", "llama3.1:8B"]
DEFAULT_WORLDS = [1, 2, 4, 8, 16]


def check_zero_layout(models=DEFAULT_MODELS, worlds=DEFAULT_WORLDS) -> list[str]:
    """Every non-expert tensor's per-layer shard intervals are equal-sized, ordered by rank, disjoint, and cover
    exactly [offset + l*size, offset + (l+1)*size); a world size that does not divide a tensor must be reported by
    ``validate_sharding`` instead of producing a layout."""
    problems = []
    for desc in models:
        cfg = config_from_descriptor(desc)
        layout = cfg.layout()
        for world in worlds:
            refused = zero.validate_sharding(cfg, world, 3)
            if refused:
                # a refusal is right when a tensor does not divide, or a shard would not be a whole number of 16-byte units
                unsplittable = [s.spec.name for s in layout.slots if not s.spec.expert and s.size % (8 * world)]
                if not unsplittable:
                    problems.append(f"{desc} P={world}: refused ({refused[0]}) although every tensor splits")
                continue
            table = zero.shard_intervals_table(cfg, world)
            for slot in layout.slots:
                if slot.spec.expert:
                    continue
                rows = table[slot.spec.name]
                if len(rows) != slot.layers * world:
                    problems.append(f"{desc} P={world} {slot.spec.name}: {len(rows)} intervals, expected {slot.layers * world}")
                    continue
                for l in range(slot.layers):
                    cursor = slot.offset + l * slot.size
                    for r in range(world):
                        layer, rank, start, end = rows[l * world + r]
                        if (layer, rank) != (l, r) or start != cursor or end - start != slot.size // world:
                            problems.append(f"{desc} P={world} {slot.spec.name} layer {l} rank {r}: [{start},{end}) breaks the tiling at {cursor}")
                        cursor = end
                    if cursor != slot.offset + (l + 1) * slot.size:
                        problems.append(f"{desc} P={world} {slot.spec.name} layer {l}: shards end at {cursor}")
    return problems


def check_checkpoint(directory: str, step: int | None = None) -> list[str]:
    """The model file's header describes a known configuration and its payload has exactly the size the layout gives;
    every rank's state file is present with a matching header; the DONE marker exists."""
    problems = []
    if step is None:
        step = formats.find_max_step(directory)
        if step < 0:
            return [f"no finished checkpoint (DONE_*) in {directory}"]
    model_path, _, done_path = formats.checkpoint_paths(directory, step, 0)
    if not os.path.exists(done_path):
        problems.append(f"missing {os.path.basename(done_path)}")
    if not os.path.exists(model_path):
        return problems + [f"missing {os.path.basename(model_path)}"]
    try:
        cfg, fp32 = formats.config_from_model_header(formats.read_header(model_path), model_path)
    except formats.FormatError as e:
        return problems + [str(e)]
    want = 1024 + cfg.num_parameters() * (4 if fp32 else 2)
    have = os.path.getsize(model_path)
    if have != want:
        problems.append(f"{os.path.basename(model_path)}: {have} bytes, the header's configuration needs {want}")
    _, state0, _ = formats.checkpoint_paths(directory, step, 0)
    if not os.path.exists(state0):
        return problems + [f"missing {os.path.basename(state0)}"]
    h = formats.read_header(state0)
    if int(h[0]) != formats.state_magic(cfg.family):
        problems.append(f"{os.path.basename(state0)}: magic {int(h[0])} is not the {cfg.family} state magic")
    nproc = int(h[2])
    for rank in range(nproc):
        _, sp, _ = formats.checkpoint_paths(directory, step, rank)
        if not os.path.exists(sp):
            problems.append(f"missing {os.path.basename(sp)} (the checkpoint was written by {nproc} processes)")
            continue
        hr = formats.read_header(sp)
        if int(hr[2]) != nproc or int(hr[3]) != rank or int(hr[10]) != step:
            problems.append(f"{os.path.basename(sp)}: header says nproc {int(hr[2])} rank {int(hr[3])} step {int(hr[10])}")
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm_kittens_b200.cli.check", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("log")
    p.add_argument("path")
    p.add_argument("--final-step", type=int)
    p.add_argument("--max-train-loss", type=float)
    p.add_argument("--max-val-loss", type=float)
    p.add_argument("--no-decrease", action="store_true")
    p = sub.add_parser("compare")
    p.add_argument("a")
    p.add_argument("b")
    p.add_argument("--rel-tol", type=float, default=0.02)
    p.add_argument("--abs-tol", type=float, default=0.02)
    p = sub.add_parser("zero-layout")
    p.add_argument("--models", nargs="*", default=DEFAULT_MODELS)
    p.add_argument("--world", nargs="*", type=int, default=DEFAULT_WORLDS)
    p = sub.add_parser("checkpoint")
    p.add_argument("directory")
    p.add_argument("--step", type=int)
    args = ap.parse_args(argv)

    if args.command == "log":
        problems = validate_log(args.path, args.final_step, args.max_train_loss, args.max_val_loss, not args.no_decrease)
    elif args.command == "compare":
        problems = compare_logs(args.a, args.b, args.rel_tol, args.abs_tol)
    elif args.command == "zero-layout":
        problems = check_zero_layout(args.models, args.world)
    else:
        problems = check_checkpoint(args.directory, args.step)
    for line in problems:
        print("FAIL:", line)
    if not problems:
        print("ok")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
