"""Launch recipes: every preset parses with the trainer's own flag parser and carries the hyper-parameters of the
reference's launch script of the same name (scripts/run_gpt2_124M.sh:44-63 and its siblings)."""
import pytest

from llm_kittens_b200.cli import flags, recipes

# (recipe, trainer, -e, B, T, tokens per step, zero, recompute, lr, final lr fraction, warmup, weight decay, checkpoint every, steps)
EXPECTED = [
    ("gpt2_124M", "gpt2", "d12", 64, 1024, 524288, 1, 0, 6e-4, 0.0, 700, 0.1, 5000, 18865),
    ("gpt2_350M", "gpt2", "d24", 64, 1024, 524288, 1, 0, 3e-4, 0.0, 700, 0.1, 2000, 60000),
    ("gpt2_774M", "gpt2", "d36", 32, 1024, 524288, 1, 0, 2.5e-4, 0.0, 700, 0.1, 4000, 286102),
    ("gpt2_1558M", "gpt2", "d48", 16, 1024, 1048576, 1, 0, 6e-4, 0.1, 700, 0.1, 2000, 32000),
    ("gpt3_125M", "gpt2", "gpt3:c768", 32, 2048, 524288, 1, 0, 6e-4, 0.1, 700, 0.1, 10000, 572204),
    ("llama3_1B", "llama3", "llama3:1B", 32, 2048, 524288, 1, 0, 3e-4, 0.1, 2000, 0.1, 5000, 57220),
    ("gpt2_124M_2nodes", "gpt2", "d12", 64, 1024, 2097152, 1, 0, 6e-4, 0.0, 700, 0.1, 5000, 18865),
    ("llama3_8B", "llama3", "llama3:8B", 4, 2048, 524288, 2, 1, 3e-4, 0.1, 2000, 0.1, 5000, 57220),
]


def test_every_recipe_is_covered():
    assert sorted(r[0] for r in EXPECTED) == sorted(recipes.RECIPES)


@pytest.mark.parametrize("name,trainer,model,B,T,D,zero,rec,lr,q,warm,wd,ckpt,steps", EXPECTED)
def test_recipe_flags(name, trainer, model, B, T, D, zero, rec, lr, q, warm, wd, ckpt, steps):
    r = recipes.RECIPES[name]
    assert r.trainer == trainer
    a = flags.parse_flags(recipes.trainer_flags(r), trainer)
    assert (a.load_filename, a.B, a.T, a.total_batch_size, a.zero_stage, a.recompute) == (model, B, T, D, zero, rec)
    assert a.learning_rate == pytest.approx(lr) and a.final_learning_rate_frac == pytest.approx(q)
    assert (a.warmup_iterations, a.checkpoint_every, a.max_steps) == (warm, ckpt, steps)
    assert a.weight_decay == pytest.approx(wd) and a.hellaswag_eval == 1 and a.val_loss_every == 250
    assert D % (B * T * 8 * r.nodes) == 0      # whole micro-steps on the node count the preset was written for
    assert a.output_log_dir == r.out_dir


def test_overrides_and_extra_flags_win():
    r = recipes.RECIPES["gpt2_350M"]
    a = flags.parse_flags(recipes.trainer_flags(r, out_dir="run7", max_steps=100, train="t_*.bin", val="v_*.bin",
                                                extra=["-z", "3", "-r", "2"]), "gpt2")
    assert (a.output_log_dir, a.max_steps, a.train_data_pattern, a.val_data_pattern) == ("run7", 100, "t_*.bin", "v_*.bin")
    assert (a.zero_stage, a.recompute) == (3, 2)
    with pytest.raises(flags.FlagError):
        recipes.trainer_flags(recipes.RECIPES["llama3_1B"], extra=["-ge", "1"])    # the Llama trainer has no -ge


def test_torchrun_command_and_dry_run(capsys):
    r = recipes.RECIPES["gpt2_124M"]
    cmd = recipes.torchrun_command(r, recipes.trainer_flags(r), gpus=4, nnodes=2, node_rank=1, master_addr="10.0.0.1", master_port=1234)
    assert cmd[1:4] == ["-m", "torch.distributed.run", "--nnodes=2"] and "--node-rank=1" in cmd and "--nproc-per-node=4" in cmd
    assert cmd[cmd.index("--master-addr") + 1] == "10.0.0.1" and "llm_kittens_b200.cli.train_gpt2cu" in cmd
    assert recipes.main(["gpt2_124M", "--gpus", "2", "--dry-run", "--", "-x", "10"]) == 0
    out = capsys.readouterr().out
    assert "--nproc-per-node=2" in out and out.rstrip().endswith("-x 10")
    assert recipes.main(["list"]) == 0 and "llama3_8B" in capsys.readouterr().out
    assert recipes.main(["nope"]) == 2


def test_scheduler_launchers_build_the_rendezvous_flags():
    env = {"SLURM_NTASKS": "16", "SLURM_PROCID": "9", "SLURM_NTASKS_PER_NODE": "8(x2)"}
    assert recipes.rendezvous_flags("slurm", "fs", fs_path="/shared/x", env=env) == ["-pn", "16", "-pr", "9", "-pg", "8", "-pi", "fs",
                                                                                      "-pf", "/shared/x"]
    assert recipes.rendezvous_flags("slurm", "tcp", server_ip="10.0.1.220", env=env)[-4:] == ["-pi", "tcp", "-ps", "10.0.1.220"]
    mpi = {"OMPI_COMM_WORLD_SIZE": "16", "OMPI_COMM_WORLD_RANK": "3", "OMPI_COMM_WORLD_LOCAL_SIZE": "8"}
    assert recipes.rendezvous_flags("mpi", "mpi", env=mpi) == ["-pn", "16", "-pr", "3", "-pg", "8", "-pi", "mpi"]
    assert recipes.rendezvous_flags("mpi", "mpi", server_ip="10.0.0.5", env=mpi)[-2:] == ["-ps", "10.0.0.5"]
    with pytest.raises(ValueError):
        recipes.rendezvous_flags("slurm", "tcp", env=env)            # no server address
    with pytest.raises(ValueError):
        recipes.rendezvous_flags("slurm", "fs", fs_path="/x", env={})   # not inside a job
    # the flags pass the trainer's parser together with a preset
    a = flags.parse_flags(recipes.trainer_flags(recipes.RECIPES["llama3_8B"], extra=recipes.rendezvous_flags("mpi", "mpi", env=mpi)), "llama3")
    assert (a.num_processes, a.process_rank, a.gpus_per_node, a.nccl_init_method) == (16, 3, 8, "mpi")


def test_scheduler_task_runs_the_trainers_dry_run(monkeypatch, capsys):
    """One task of a (pretended) 16-task slurm job: the preset goes through the trainer's host-only dry run (-x 0)."""
    for k, v in (("SLURM_NTASKS", "16"), ("SLURM_PROCID", "9"), ("SLURM_NTASKS_PER_NODE", "8")):
        monkeypatch.setenv(k, v)
    rc = recipes.main(["gpt2_124M_2nodes", "--launcher", "slurm", "--rendezvous", "tcp", "--server-ip", "127.0.0.1", "--", "-x", "0"])
    assert rc == 0
    assert "ZeRO-1 layout validated for 16 process(es)" in capsys.readouterr().out
