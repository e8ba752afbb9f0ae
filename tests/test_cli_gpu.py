"""End-to-end trainer CLI on the GPU: synthetic shards, checkpoint at step 3, resume, bit-identical continuation."""
import os
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _train(args, cwd):
    cmd = [sys.executable, "-m", "llm_kittens_b200.cli.train_gpt2cu", *args]
    r = subprocess.run(cmd, cwd=cwd, env=dict(os.environ, PYTHONPATH=REPO), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-2000:])
    return r.stdout


def test_train_checkpoint_resume_is_bit_exact(tmp_path):
    from llm_kittens_b200.data import prepare
    from llm_kittens_b200.utils.logger import parse_log

    prepare.prepare_synthetic(str(tmp_path / "data"), 400_000, vocab_size=50257, seed=3)
    common = ["-i", str(tmp_path / "data" / "synthetic_train_*.bin"), "-j", str(tmp_path / "data" / "synthetic_val_*.bin"),
              "-e", "d6", "-b", "4", "-t", "64", "-d", "512", "-x", "6", "-l", "1e-3", "-u", "2", "-q", "0.1", "-c", "0.1",
              "-v", "3", "-m", "2", "-s", "0", "-h", "0", "-r", "0"]
    run_a = tmp_path / "a"
    _train([*common, "-o", str(run_a), "-n", "3"], str(tmp_path))
    assert os.path.exists(run_a / "DONE_00000003") and os.path.exists(run_a / "model_00000003.bin")
    full = parse_log(str(run_a / "main.log"))
    assert len(full["train"]) == 6
    # continue from the step-3 checkpoint in a copy of the directory
    run_b = tmp_path / "b"
    shutil.copytree(run_a, run_b)
    for name in os.listdir(run_b):
        if "00000006" in name:
            os.remove(run_b / name)
    _train([*common, "-o", str(run_b), "-n", "3", "-y", "1"], str(tmp_path))
    resumed = parse_log(str(run_b / "main.log"))
    steps = sorted(full["train"])
    later = steps[3:]                      # the steps after the checkpoint
    assert later and all(s in resumed["train"] for s in later)
    for s in later:                        # loss, learning rate and gradient norm as logged: identical digits
        assert resumed["train"][s] == full["train"][s], (s, resumed["train"][s], full["train"][s])


def test_device_preflight_passes_on_this_machine(capsys):
    from llm_kittens_b200.cli import check

    assert check.main(["device"]) == 0
    out = capsys.readouterr().out
    assert "sm_100" in out and "resident CTA pairs" in out and out.rstrip().endswith("ok")
