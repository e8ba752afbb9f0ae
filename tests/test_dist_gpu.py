"""Two-GPU tests (skipped when fewer than two GPUs are visible): the fused peer-memory communication
path must train like the library-collective path and like ZeRO-0, within bf16 tolerance."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def _need_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


def _run(mode, tmp_path, **env):
    from test_dist_cpu import launch

    d = tmp_path / (mode + "".join(f"_{k}{v}" for k, v in env.items()))
    d.mkdir()
    outs = launch(mode, d, extra_env={"NCCL_NVLS_ENABLE": "0", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "1", **env})
    for rc, out in outs:
        assert rc == 0, out[-3000:]
    return torch.load(d / "rank0.pt"), torch.load(d / "rank1.pt")


def test_fused_comm_matches_library_and_zero0(tmp_path):
    _need_two_gpus()
    f0, f1 = _run("gpu_fused", tmp_path)
    l0, l1 = _run("gpu_library1", tmp_path)
    z0, _ = _run("gpu_library0", tmp_path)
    assert torch.equal(f0["params"], f1["params"]) and torch.equal(l0["params"], l1["params"])
    for a, b, c in zip(f0["losses"], l0["losses"], z0["losses"]):
        assert abs(a - b) < 0.02 and abs(a - c) < 0.02
    for a, b in zip(f0["norms"], l0["norms"]):
        assert abs(a - b) < 0.03 * max(1.0, b)
    assert (f0["params"] - l0["params"]).abs().max().item() < 0.02
    assert f0["losses"][-1] < f0["losses"][0]


def test_fused_comm_with_replicated_state_matches_library_zero0(tmp_path):
    """ZeRO-0 on the framework's own kernels: every rank averages all copies of every gradient by peer loads and
    updates all parameters itself; same training as the NCCL all-reduce path, replicas bit-identical."""
    _need_two_gpus()
    f0, f1 = _run("gpu_fused0", tmp_path)
    z0, _ = _run("gpu_library0", tmp_path)
    assert torch.equal(f0["params"], f1["params"])
    assert f0["losses"] == f1["losses"] and f0["norms"] == f1["norms"]
    for a, b in zip(f0["losses"], z0["losses"]):
        assert abs(a - b) < 0.02
    for a, b in zip(f0["norms"], z0["norms"]):
        assert abs(a - b) < 0.03 * max(1.0, b)
    assert (f0["params"] - z0["params"]).abs().max().item() < 0.02


def test_fused_comm_micro_step_replayed_from_cuda_graphs(tmp_path):
    """The fused ZeRO-1 micro-step (forward, backward, per-bucket signals and reduce-scatter kernels that read the
    step's epoch from device memory) captured once and replayed: the same losses, norms and parameters as eager
    launches, bit for bit (the kernels and their order are the same)."""
    _need_two_gpus()
    e0, e1 = _run("gpu_fused", tmp_path)
    g0, g1 = _run("gpu_fused", tmp_path, LLMK_TEST_GRAPH="1")
    assert torch.equal(g0["params"], g1["params"])
    assert g0["losses"] == e0["losses"] and g0["norms"] == e0["norms"]
    assert torch.equal(g0["params"], e0["params"])


def test_fused_comm_survives_a_skipped_update(tmp_path):
    """A step without optimizer update (z-score guards) must still raise the "parameters ready" flag: the steps
    after it run without a bounded wait running out (the worker checks the status word) and train like the library
    path that skips the same step."""
    _need_two_gpus()
    f0, f1 = _run("gpu_fused", tmp_path, LLMK_TEST_SKIP_STEP="1")
    l0, _ = _run("gpu_library1", tmp_path, LLMK_TEST_SKIP_STEP="1")
    assert torch.equal(f0["params"], f1["params"])
    for a, b in zip(f0["losses"], l0["losses"]):
        assert abs(a - b) < 0.02
    assert (f0["params"] - l0["params"]).abs().max().item() < 0.02


def test_expert_parallel_moe_matches_single_process(tmp_path):
    _need_two_gpus()
    from dist_worker import global_batches, tiny_moe_config
    from llm_kittens_b200.models.moe import MoETransformer
    from llm_kittens_b200.runtime.trainer import Trainer

    cfg = tiny_moe_config()
    model = MoETransformer(cfg, device="cuda:0", recompute=0)
    model.init_weights(42)
    tr = Trainer(model, learning_rate=1e-3, weight_decay=0.1)
    ref = []
    for x, y in global_batches(cfg, 3, 2, 2, 128):
        ref.append(tr.train_step([(x[:2].contiguous(), y[:2].contiguous()), (x[2:].contiguous(), y[2:].contiguous())]).loss)
    for mode, env in (("gpu_moe_library1", {}), ("gpu_moe_fused", {}), ("gpu_moe_a2a1", {}),
                      ("gpu_moe_fused", {"LLMK_MOE_RETURN": "scatter", "LLMK_MOE_DISPATCH": "push"}),
                      ("gpu_moe_fused", {"LLMK_MOE_RETURN": "push", "LLMK_MOE_DISPATCH": "push"})):
        r0, r1 = _run(mode, tmp_path, **env)
        assert r0["losses"] == r1["losses"]
        for a, b in zip(r0["losses"], ref):
            assert abs(a - b) < 0.03, (mode, r0["losses"], ref)
        assert r0["losses"][-1] < r0["losses"][0]


@pytest.mark.parametrize("stage,recompute,gather", [(2, 0, ""), (3, 0, ""), (3, 3, ""), (3, 0, "chunks"), (3, 3, "chunks"), (3, 0, "bucket")])
def test_sharded_zero_stages_match_library(tmp_path, stage, recompute, gather):
    """Really sharded gradients (stage 2) and parameters (stage 3), two micro-steps per step, four blocks
    (so that the two bucket slots are reused inside a micro-step): same training as the library path. Stage 3
    gathers a block's weight matrices chunk by chunk while the GEMMs poll the chunk flags: run with the default chunk
    size (one chunk per shard at this model size), with 8 KiB chunks (several flags per matrix, tiles that span
    two chunks) and with the bucket-granular gather."""
    _need_two_gpus()
    env = {"LLMK_TEST_LAYERS": "4", "LLMK_TEST_RECOMPUTE": str(recompute)}
    if gather == "chunks":
        env["LLMK_AG_CHUNK_BYTES"] = "8192"
    elif gather == "bucket":
        env["LLMK_AG_FLAGS"] = "0"
    s0, s1 = _run(f"gpu_sharded{stage}", tmp_path, **env)
    l0, _ = _run("gpu_library1", tmp_path, LLMK_TEST_LAYERS="4", LLMK_TEST_RECOMPUTE=str(recompute))
    assert torch.equal(s0["params"], s1["params"])
    assert s0["losses"] == s1["losses"]
    for a, b in zip(s0["losses"], l0["losses"]):
        assert abs(a - b) < 0.02, (s0["losses"], l0["losses"])
    for a, b in zip(s0["norms"], l0["norms"]):
        assert abs(a - b) < 0.03 * max(1.0, b)
    assert (s0["params"] - l0["params"]).abs().max().item() < 0.02
    assert s0["losses"][-1] < s0["losses"][0]


def test_cli_zero3_checkpoint_resume_two_gpus(tmp_path):
    """Trainer CLI on two GPUs with really sharded parameters: checkpoint (a collective gather of the shards),
    resume from it, and a bit-identical continuation of the logged losses."""
    _need_two_gpus()
    import shutil
    import subprocess

    from llm_kittens_b200.data import prepare
    from llm_kittens_b200.utils.logger import parse_log
    from test_dist_cpu import free_port

    repo = os.path.dirname(HERE)
    prepare.prepare_synthetic(str(tmp_path / "data"), 400_000, vocab_size=50257, seed=3)
    common = ["-i", str(tmp_path / "data" / "synthetic_train_*.bin"), "-j", str(tmp_path / "data" / "synthetic_val_*.bin"),
              "-e", "d6", "-b", "4", "-t", "64", "-d", "1024", "-x", "6", "-l", "1e-3", "-u", "2", "-q", "0.1", "-c", "0.1",
              "-v", "3", "-m", "2", "-s", "0", "-h", "0", "-r", "0", "-z", "3", "-n", "3"]

    def run(out_dir, extra):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
               "--master-port", str(free_port()), "-m", "llm_kittens_b200.cli.train_gpt2cu", *common, "-o", str(out_dir), *extra]
        env = dict(os.environ, PYTHONPATH=repo, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
        r = subprocess.run(cmd, cwd=str(tmp_path), env=env, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-3000:])
        return r.stdout

    a = tmp_path / "a"
    out = run(a, [])
    assert "ShardedComm" in out
    full = parse_log(str(a / "main.log"))["train"]
    assert len(full) == 6 and os.path.exists(a / "DONE_00000003") and os.path.exists(a / "state_00000003_00001.bin")
    b = tmp_path / "b"
    shutil.copytree(a, b)
    for name in os.listdir(b):
        if "00000006" in name:
            os.remove(b / name)
    run(b, ["-y", "1"])
    resumed = parse_log(str(b / "main.log"))["train"]
    for s in sorted(full)[3:]:
        assert resumed[s] == full[s], (s, resumed[s], full[s])


def test_rank_that_leaves_between_steps_is_noticed_on_the_host(tmp_path):
    """The same scenario on two GPUs with NCCL (NVLS off): rank 1 leaves between steps with nothing in flight, rank 0
    finds out at the host-side rendezvous before it launches step 2 and exits with the resume code."""
    _need_two_gpus()
    from test_dist_cpu import launch

    from llm_kittens_b200.runtime.watchdog import EXIT_RESUME

    outs = launch("gpu_leave1", tmp_path, extra_env={"NCCL_NVLS_ENABLE": "0", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "1"}, timeout=240)
    assert outs[1][0] == 0, outs[1][1][-2000:]
    assert outs[0][0] == EXIT_RESUME, outs[0][1][-2000:]
    r0, r1 = torch.load(tmp_path / "rank0.pt"), torch.load(tmp_path / "rank1.pt")
    assert r1["outcome"] == "left" and r0["outcome"] == "peer_left"
    assert len(r0["losses"]) == 2 and r0["losses"] == r1["losses"]


@pytest.mark.parametrize("hs", [64, 128])
def test_context_parallel_attention_matches_the_full_sequence(tmp_path, hs):
    """Two ranks, each with one chunk of the sequence, keys and values pulled from the peer's memory by the attention
    kernels themselves: outputs and QKV gradients of every chunk equal the single-GPU kernels on the whole sequence
    (forward 0.03, backward 0.08 like the attention tests), and a second call gives the same bits."""
    _need_two_gpus()
    r0, r1 = _run(f"gpu_cp{hs}", tmp_path)
    T = r0["out"].shape[1]
    for r, res in enumerate((r0, r1)):
        assert res["same"]
        ref_o, ref_d = r0["ref_out"][:, r * T:(r + 1) * T], r0["ref_dqkv"][:, r * T:(r + 1) * T]
        assert (res["out"] - ref_o).abs().max().item() < 0.03
        assert (res["dqkv"] - ref_d).abs().max().item() < 0.08


def test_two_devices_in_one_process():
    """Function attributes (opt-in shared memory) and cached device properties are per device: a process that has
    used the kernels on cuda:0 must be able to use them on cuda:1 as well (GEMM, attention, norm backward, classifier:
    the launchers that need more than the default shared memory)."""
    _need_two_gpus()
    from llm_kittens_b200.ops import _native, attention, classifier, gemm, norm

    results = []
    for dev in (0, 1, 0):
        with torch.cuda.device(dev):
            g = torch.Generator(device=f"cuda:{dev}").manual_seed(3)
            rnd = lambda *s: (torch.randn(*s, generator=g, device=f"cuda:{dev}") * 0.1).to(torch.bfloat16)
            a, w, bias = rnd(512, 256), rnd(768, 256), rnd(768)
            out = gemm.gemm_nt(a, w, bias=bias)
            pre = torch.empty_like(out)
            act = gemm.gemm_nt(a, w, bias=bias, gelu_pre_out=pre)
            dw = gemm.gemm_tn(out, a)
            qkv = rnd(1, 256, 3 * 4 * 64)
            o, lse = attention.attention_fwd(qkv, 1, 256, 4, 4, 64)
            dqkv = attention.attention_bwd(rnd(1, 256, 4 * 64), qkv, o, lse, 1, 256, 4, 4, 64)
            x, lw, lb = rnd(512, 768), rnd(768) + 1, rnd(768)
            ln, mean, rstd = norm.layernorm_fwd(x, lw, lb)
            dinp, dlw, dlb = torch.zeros_like(x), torch.zeros_like(lw), torch.zeros_like(lb)
            norm.layernorm_bwd(dinp, dlw, dlb, ln, x, lw, mean, rstd)
            logits = rnd(64, 50304)
            tg = torch.randint(0, 50257, (64,), generator=g, device=f"cuda:{dev}", dtype=torch.int32)
            losses = classifier.fused_classifier(logits, tg, 50257, 1.0 / 64)
            torch.cuda.synchronize()
            _native.check_status()
            results.append([t.float().cpu() for t in (out, act, dw, o, dqkv, dinp, losses)])
    for a, b in zip(results[0], results[1]):
        assert torch.equal(a, b)      # the same seeded inputs give the same bits on both devices
    for a, b in zip(results[0], results[2]):
        assert torch.equal(a, b)
