"""Checkpoint write / resume / pruning.

Directory protocol of the reference (train_gpt2.cu:1569-1604, 2196-2210): rank 0 writes
``model_%08d.bin`` (world-size independent), every rank writes ``state_%08d_%05d.bin`` (its optimizer
shard, RNG and loader position), then after a barrier rank 0 creates the empty marker ``DONE_%08d``.
A checkpoint without its DONE marker is ignored on resume. Resume restores m / v / master, re-derives
the bf16 parameters from the master copy with the rounding noise of the last update (so the restart
continues bit-exactly), and puts the data loader back at its shard / sample position including the
shuffle permutations and the MT19937 state.
"""
from __future__ import annotations

import os

from ..utils import formats


def save_checkpoint(output_dir: str, step: int, trainer, loader, world: int, rank: int, comm=None) -> None:
    os.makedirs(output_dir, exist_ok=True)
    model_path, state_path, done_path = formats.checkpoint_paths(output_dir, step, rank)
    cfg = trainer.model.config
    params = trainer.full_params()   # a collective when the parameters are sharded: every rank takes part
    if rank == 0:
        formats.write_model(model_path, cfg, params)
    del params
    formats.write_state(state_path, cfg.family, world, rank, step, trainer.m, trainer.v, trainer.master,
                        trainer.rng.state, trainer.rng_state_last_update,
                        loader.current_shard_idx if loader is not None else 0,
                        loader.current_sample_idx if loader is not None else 0,
                        loader.shuffle_state() if loader is not None else b"")
    if comm is not None:
        comm.barrier()
    if rank == 0:
        open(done_path, "w").close()


def load_checkpoint(output_dir: str, step: int, trainer, loader, world: int, rank: int) -> int:
    """Restore trainer (and loader) from the checkpoint of ``step``; returns the step to continue at.
    The model parameters must already have been loaded from ``model_%08d.bin``."""
    _, state_path, done_path = formats.checkpoint_paths(output_dir, step, rank)
    if not os.path.exists(done_path):
        raise FileNotFoundError(f"checkpoint {step} in {output_dir} has no DONE marker")
    info = formats.read_state(state_path, trainer.model.config.family, world, rank, trainer.m, trainer.v, trainer.master)
    trainer.rng.state = info["rng_state"]
    trainer.rng_state_last_update = info["rng_state_last_update"]
    trainer.step_count = info["step"]
    if trainer.use_master:
        trainer.restore_params_from_master()
    if loader is not None:
        loader.resume(info["shard_idx"], info["sample_idx"], info["shuffle_blob"])
    return info["step"]


def prune_checkpoints(output_dir: str, step: int, every: int, keep: int, major_every: int, world: int, rank: int) -> None:
    """Keep the last ``keep`` checkpoints (0 = keep all); steps that are multiples of ``major_every`` stay."""
    if keep <= 0 or every <= 0:
        return
    victim = step - keep * every
    if victim <= 0:
        return
    if major_every > 0 and victim % major_every == 0:
        return
    model_path, state_path, done_path = formats.checkpoint_paths(output_dir, victim, rank)
    if rank == 0:
        for p in (done_path, model_path):
            if os.path.exists(p):
                os.remove(p)
    if os.path.exists(state_path):
        os.remove(state_path)
