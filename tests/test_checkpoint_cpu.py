"""Checkpoint protocol on CPU (oracle model): model / state / DONE files, resume continues exactly
where an uninterrupted run would be (same losses, same batches), pruning keeps the last k and the
major checkpoints. Mirrors the save -> reload -> identical-losses check of the reference's
test_gpt2.cu:349-390."""
import os

import numpy as np
import torch

from llm_kittens_b200.models.config import ModelConfig
from llm_kittens_b200.oracle.torch_model import TorchTransformer
from llm_kittens_b200.runtime.checkpoint import load_checkpoint, prune_checkpoints, save_checkpoint
from llm_kittens_b200.runtime.trainer import Trainer
from llm_kittens_b200.utils import formats
from llm_kittens_b200.utils.dataloader import DataLoader


def cfg_tiny():
    return ModelConfig(family="gpt2", max_seq_len=32, vocab_size=256, padded_vocab_size=256, num_layers=2, num_heads=2,
                       num_kv_heads=2, channels=64, hidden_dim=256)


def make(tmp_path, seed=42):
    cfg = cfg_tiny()
    model = TorchTransformer(cfg, device="cpu", dtype=torch.float32)
    model.init_weights(seed)
    tr = Trainer(model, learning_rate=1e-2, weight_decay=0.1)
    loader = DataLoader(str(tmp_path / "train_*.bin"), 2, 32, 0, 1, should_shuffle=True, ring=3)
    return cfg, model, tr, loader


def test_resume_is_exact_and_files_follow_the_protocol(tmp_path):
    rng = np.random.default_rng(0)
    for i in range(2):
        formats.write_tokens(str(tmp_path / f"train_{i}.bin"), rng.integers(0, 256, size=2000))
    out = str(tmp_path / "log")
    cfg, model, tr, loader = make(tmp_path)
    losses = []
    for step in range(10):
        if step == 5:
            save_checkpoint(out, step, tr, loader, 1, 0)
        x, y = loader.next_batch()
        losses.append(tr.train_step([(x, y)]).loss)
    assert sorted(os.listdir(out)) == ["DONE_00000005", "model_00000005.bin", "state_00000005_00000.bin"]
    assert formats.find_max_step(out) == 5
    h = formats.read_header(os.path.join(out, "state_00000005_00000.bin"))
    assert list(h[:6]) == [20240527, 1, 1, 0, 0, 1] and h[10] == 5   # fp32 model: no master copy; shuffle state present
    # fresh process state: new model from the checkpoint file, new trainer, new loader
    cfg2, flat = formats.read_model(os.path.join(out, "model_00000005.bin"), dtype=torch.float32)
    _, model2, tr2, loader2 = make(tmp_path, seed=7)
    model2.load_parameters(flat)
    step = load_checkpoint(out, 5, tr2, loader2, 1, 0)
    assert step == 5 and tr2.step_count == tr.step_count - 5
    for s in range(5, 10):
        x, y = loader2.next_batch()
        assert tr2.train_step([(x, y)]).loss == losses[s]
    assert torch.equal(model2.params, model.params)


def test_missing_done_marker_and_pruning(tmp_path):
    rng = np.random.default_rng(0)
    formats.write_tokens(str(tmp_path / "train_0.bin"), rng.integers(0, 256, size=2000))
    out = str(tmp_path / "log")
    cfg, model, tr, loader = make(tmp_path)
    for step in (10, 20, 30, 40):
        save_checkpoint(out, step, tr, loader, 1, 0)
        prune_checkpoints(out, step, every=10, keep=2, major_every=20, world=1, rank=0)
    names = sorted(os.listdir(out))
    # step 10 pruned when 30 was written; step 20 is "major" and survives; 30 and 40 are the last two
    assert "DONE_00000010" not in names and "model_00000010.bin" not in names and "state_00000010_00000.bin" not in names
    for s in (20, 30, 40):
        assert "DONE_%08d" % s in names
    os.remove(os.path.join(out, "DONE_00000040"))
    assert formats.find_max_step(out) == 30
    try:
        load_checkpoint(out, 40, tr, loader, 1, 0)
        raise AssertionError("a checkpoint without its DONE marker must be refused")
    except FileNotFoundError:
        pass
