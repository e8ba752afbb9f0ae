"""Tensor / sequence / pipeline / context parallel primitives on gloo ranks (CPU)."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def launch(mode, out_dir, world):
    from test_dist_cpu import free_port

    port = free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "primitives_worker.py"), mode, str(out_dir)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    for p in procs:
        out, _ = p.communicate(timeout=240)
        assert p.returncode == 0, out[-3000:]
    return [torch.load(os.path.join(out_dir, f"rank{r}.pt")) for r in range(world)]


def test_tensor_parallel_mlp_matches_full(tmp_path):
    world = 2
    res = launch("tp", tmp_path, world)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(6, 16, generator=g)
    w1, b1 = torch.randn(32, 16, generator=g), torch.randn(32, generator=g)
    w2 = torch.randn(16, 32, generator=g)
    dy = torch.randn(6, 16, generator=g)
    h = x @ w1.t() + b1
    y = h @ w2.t()
    dh = dy @ w2
    for r in range(world):
        assert torch.allclose(res[r]["y"], y, atol=1e-4)
        assert torch.allclose(res[r]["dx"], dh @ w1, atol=1e-4)
        assert torch.allclose(res[r]["dw1s"], (dh.t() @ x).chunk(world)[r], atol=1e-4)
        assert torch.allclose(res[r]["db1s"], dh.sum(0).chunk(world)[r], atol=1e-4)
        assert torch.allclose(res[r]["dw2s"], (dy.t() @ h).chunk(world, dim=1)[r], atol=1e-4)


def test_sequence_parallel_and_all_to_all(tmp_path):
    world = 2
    res = launch("sp", tmp_path, world)
    for r in range(world):
        assert torch.equal(res[r]["gathered"], res[r]["full"])
        assert torch.allclose(res[r]["back"], world * res[r]["full"].chunk(world, dim=1)[r])
        expect = torch.cat([torch.arange(r * 2, r * 2 + 2, dtype=torch.float32) + 100 * s for s in range(world)])
        assert torch.equal(res[r]["a2a"], expect)


def test_one_f_one_b_schedule_properties():
    from llm_kittens_b200.parallel.primitives import one_f_one_b_schedule

    for stages in (1, 2, 4):
        for micro in (1, 3, 8):
            for st in range(stages):
                ops = one_f_one_b_schedule(stages, micro, st)
                assert sorted(o.micro for o in ops if o.kind == "F") == list(range(micro))
                assert [o.micro for o in ops if o.kind == "B"] == list(range(micro))
                alive = peak = 0
                done_f = set()
                for o in ops:
                    if o.kind == "F":
                        alive += 1
                        done_f.add(o.micro)
                    else:
                        assert o.micro in done_f
                        alive -= 1
                    peak = max(peak, alive)
                assert peak <= stages - st


def test_pipeline_two_stages_matches_single_process(tmp_path):
    world = 2
    res = launch("pp", tmp_path, world)
    assert abs(res[1]["loss"] - res[0]["ref_loss"]) < 1e-5
    for r in range(world):
        for a, b in zip(res[r]["grads"], res[0]["ref_grads"][r]):
            assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.parametrize("world", [2, 3])
def test_ring_attention_matches_full_causal_attention(tmp_path, world):
    res = launch("ring", tmp_path, world)
    for r in range(world):
        d = res[r]
        assert torch.allclose(d["out"], d["ref"], atol=1e-5)
        for a, b in (("dq", "rdq"), ("dk", "rdk"), ("dv", "rdv")):
            assert torch.allclose(d[a], d[b], atol=1e-4), (r, a)


def test_expert_parameters_are_gathered_from_their_owners_for_a_checkpoint(tmp_path):
    """Library back-end with expert parallelism: a rank never updates (or reads) another rank's experts, so before the
    model file is written every expert is broadcast from its owner (``LibraryComm.gather_expert_params``, called by
    ``Trainer.full_params``)."""
    res = launch("experts", tmp_path, 2)
    for r in res:
        assert r["experts"] > 0
        assert torch.equal(r["params"], r["want"])
    assert torch.equal(res[0]["params"], res[1]["params"])
