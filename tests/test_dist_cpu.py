"""Multi-process tests of the ZeRO / trainer logic on CPU ranks (gloo, world size 2): every stage must
train exactly like one process that sees the whole global batch; a rank that fails on the host is
detected by the others through the process-group timeout (no GPU involved)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def launch(mode, out_dir, world=2, extra_env=None, timeout=420):
    port = free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   LOCAL_RANK=str(r), OMP_NUM_THREADS="2")
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "dist_worker.py"), mode, str(out_dir)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append((p.returncode, out))
    return outs


def single_process_reference(steps=4, skip_step=-1):
    sys.path.insert(0, HERE)
    from dist_worker import global_batches, tiny_config
    from llm_kittens_b200.oracle.torch_model import TorchTransformer
    from llm_kittens_b200.runtime.trainer import Trainer

    cfg = tiny_config()
    model = TorchTransformer(cfg, device="cpu", dtype=torch.float32)
    model.init_weights(42)
    tr = Trainer(model, learning_rate=1e-3, weight_decay=0.1)
    losses = []
    for i, (x, y) in enumerate(global_batches(cfg, steps, 2, 2, 64)):
        # two micro-batches of the rank-local size == the data-parallel average over two ranks
        micro = [(x[:2], y[:2]), (x[2:], y[2:])]
        if i == skip_step:
            tr.accumulate(micro)
            tr.update(1e-3, skip=True)
            losses.append(tr.read_scalars()[0])
            tr.skip_update()
        else:
            losses.append(tr.train_step(micro).loss)
    return losses, model.params.clone()


@pytest.mark.parametrize("stage", [0, 1, 2, 3])
def test_zero_stages_match_single_process(tmp_path, stage):
    outs = launch(f"cpu_zero{stage}", tmp_path)
    for rc, out in outs:
        assert rc == 0, out
    ref_losses, ref_params = single_process_reference()
    r0, r1 = torch.load(tmp_path / "rank0.pt"), torch.load(tmp_path / "rank1.pt")
    assert torch.equal(r0["params"], r1["params"])  # replicas stay identical
    for a, b in zip(r0["losses"], ref_losses):
        assert abs(a - b) < 1e-4
    assert r0["losses"] == r1["losses"] and r0["norms"] == r1["norms"]
    assert (r0["params"] - ref_params).abs().max().item() < 1e-5
    assert r0["losses"][-1] < r0["losses"][0]


def test_skipped_update_keeps_ranks_in_step(tmp_path):
    """Step 1 runs reduction, norm and clip but no optimizer update (what the z-score guards do): the next steps
    must run and match one process that skips the same step."""
    outs = launch("cpu_zero1", tmp_path, extra_env={"LLMK_TEST_SKIP_STEP": "1"})
    for rc, out in outs:
        assert rc == 0, out
    ref_losses, ref_params = single_process_reference(skip_step=1)
    r0, r1 = torch.load(tmp_path / "rank0.pt"), torch.load(tmp_path / "rank1.pt")
    assert torch.equal(r0["params"], r1["params"])
    for a, b in zip(r0["losses"], ref_losses):
        assert abs(a - b) < 1e-4
    assert (r0["params"] - ref_params).abs().max().item() < 1e-5


def test_non_finite_gradient_leaves_weights_and_optimizer_state_alone():
    """An inf in a gradient (injected on the host after backward) gives a non-finite norm: the update is skipped,
    reported as skipped, and nothing becomes NaN."""
    sys.path.insert(0, HERE)
    from dist_worker import global_batches, tiny_config
    from llm_kittens_b200.oracle.torch_model import TorchTransformer
    from llm_kittens_b200.runtime.trainer import Trainer

    cfg = tiny_config()
    model = TorchTransformer(cfg, device="cpu", dtype=torch.float32)
    model.init_weights(42)
    tr = Trainer(model, learning_rate=1e-3, weight_decay=0.1)
    (x, y), (x2, y2) = global_batches(cfg, 2, 1, 2, 64)
    tr.train_step([(x, y)])
    before, m_before = model.params.clone(), tr.m.clone()
    tr.accumulate([(x2, y2)])
    model.grads[5] = float("inf")
    tr.update(1e-3)
    loss, norm, bad = tr.read_scalars()
    assert bad and not torch.isfinite(torch.tensor(norm))
    assert torch.equal(model.params, before) and torch.equal(tr.m, m_before)
    r = tr.train_step([(x2, y2)])
    assert not r.skipped and r.loss == r.loss and torch.isfinite(model.params).all()


def test_failed_rank_is_detected_by_the_survivor(tmp_path):
    outs = launch("cpu_fail_rank1", tmp_path, extra_env={"LLMK_TEST_PG_TIMEOUT": "5"}, timeout=120)
    assert outs[1][0] != 0 and "injected failure" in outs[1][1]
    survivor = torch.load(tmp_path / "rank0.pt")
    assert survivor["outcome"].startswith("error:")


def test_rank_that_leaves_between_steps_is_noticed_before_the_next_launch(tmp_path):
    """Rank 1 exits cleanly after two steps; rank 0 learns of it at the host-side step rendezvous (no collective of
    step 2 is ever started) and exits with the code that the supervisor maps to a resume."""
    from llm_kittens_b200.runtime.watchdog import EXIT_RESUME

    outs = launch("cpu_leave1", tmp_path, timeout=180)
    assert outs[1][0] == 0, outs[1][1][-2000:]
    assert outs[0][0] == EXIT_RESUME, outs[0][1][-2000:]
    r0, r1 = torch.load(tmp_path / "rank0.pt"), torch.load(tmp_path / "rank1.pt")
    assert r1["outcome"] == "left" and r0["outcome"] == "peer_left"
    assert "rank(s) [1] did not enter step 2" in r0["message"]
    assert len(r0["losses"]) == 2 and r0["losses"] == r1["losses"]
