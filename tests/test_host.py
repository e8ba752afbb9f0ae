"""CPU-only tier: file formats, flag parser, dry run, ZeRO shard arithmetic, schedulers, logger and
log validators, outlier detector, RNG parity with torch, data / eval loaders on synthetic files,
tokenizer. Mirrors the reference's host-only tiers (dev/test_dataloader.cpp, dev/validate_zero_layout.py,
the -x 0 dry runs and the log validators)."""
import math
import os
import struct

import numpy as np
import pytest
import torch

from llm_kittens_b200.cli import flags as flags_mod
from llm_kittens_b200.cli import train as train_mod
from llm_kittens_b200.models.config import ModelConfig, config_from_descriptor
from llm_kittens_b200.parallel import zero
from llm_kittens_b200.utils import formats
from llm_kittens_b200.utils.dataloader import DataLoader, EvalLoader
from llm_kittens_b200.utils.logger import Logger, compare_logs, parse_log, validate_log
from llm_kittens_b200.utils.outlier import OutlierDetector
from llm_kittens_b200.utils.rand import Mt19937, Xorshift, sample_softmax
from llm_kittens_b200.utils.schedulers import LearningRateScheduler
from llm_kittens_b200.utils.tokenizer import Tokenizer


# ------------------------------------------------------------------------------------- descriptors
def test_descriptors_and_parameter_counts():
    c = config_from_descriptor("d12")
    assert (c.num_layers, c.num_heads, c.channels, c.max_seq_len) == (12, 12, 768, 1024)
    assert c.num_parameters() == 124475904  # the count the reference quotes for GPT-2 124M (best_runs.md:726)
    assert config_from_descriptor("gpt2:d48").channels == 1600
    g3 = config_from_descriptor("gpt3:c2048")
    assert (g3.num_layers, g3.num_heads, g3.max_seq_len) == (24, 16, 2048)
    l8 = config_from_descriptor("llama3:8B")
    assert l8.num_parameters() == 8030261248
    assert l8.qkv_width == 6144 and l8.hidden_dim == 14336 and not l8.tied_embeddings
    assert config_from_descriptor("llama3.1:8B").use_scaled_rope and config_from_descriptor("llama3.1:8B").max_seq_len == 8192
    l1 = config_from_descriptor("llama3.2:1B")
    assert l1.tied_embeddings and l1.head_size == 64 and l1.qkv_width == 3072
    assert l1.num_parameters() == 16 * 60821504 + 128256 * 2048 + 2048
    moe = config_from_descriptor("moe:d24")
    assert moe.family == "moe" and moe.num_experts == 8 and moe.top_k == 2 and moe.channels == 1024
    for bad in ("d13", "gpt3:c100", "llama3:70B", "foo", "gpt2:dx"):
        with pytest.raises(ValueError):
            config_from_descriptor(bad)


def test_layout_offsets_are_aligned_and_ordered():
    for d in ("d12", "gpt3:c768", "llama3:1B", "llama3.2:1B", "moe:d24"):
        lay = config_from_descriptor(d).layout()
        off = 0
        for s in lay.slots:
            assert s.offset == off and s.offset % 64 == 0
            off += s.total
        assert off == lay.total
    names = [s.spec.name for s in config_from_descriptor("d12").layout().slots]
    assert names == ["wte", "wpe", "ln1w", "ln1b", "qkvw", "qkvb", "attprojw", "attprojb", "ln2w", "ln2b", "fcw", "fcb",
                     "fcprojw", "fcprojb", "lnfw", "lnfb"]
    names = [s.spec.name for s in config_from_descriptor("llama3:1B").layout().slots]
    assert names == ["wte", "ln1w", "qkvw", "attprojw", "ln2w", "fcw_up", "fcw_gate", "fcprojw", "lnfw", "lm_head"]


# ------------------------------------------------------------------------------------- ZeRO arithmetic
@pytest.mark.parametrize("desc", ["d12", "gpt2:d24", "gpt3:c768", "gpt3:c2048", "llama3:1B", "llama3:8B", "llama3.2:1B"])
@pytest.mark.parametrize("P", [1, 2, 4, 8, 16])
def test_zero_shards_are_disjoint_contiguous_and_cover(desc, P):
    cfg = config_from_descriptor(desc)
    if zero.validate_sharding(cfg, P, 1):
        pytest.skip("not shardable at this P")
    table = zero.shard_intervals_table(cfg, P)
    lay = cfg.layout()
    for name, rows in table.items():
        slot = lay[name]
        rows = sorted(rows, key=lambda r: r[2])
        assert rows[0][2] == slot.offset and rows[-1][3] == slot.offset + slot.total
        for a, b in zip(rows, rows[1:]):
            assert a[3] == b[2]  # contiguous, disjoint
        assert all((r[3] - r[2]) == slot.size // P for r in rows)
    # per-rank plans: state buffer is total/P, segments inside the model, no overlap between ranks
    owned = np.zeros(lay.total, dtype=np.int8)
    for r in range(P):
        plan = zero.ZeroPlan(cfg, P, r, 1 if P > 1 else 0)
        assert plan.state_elements == lay.total // P
        for s in plan.segments:
            owned[s.param_off: s.param_off + s.length] += 1
            assert 0 <= s.state_off and s.state_off + s.length <= plan.state_elements
    assert (owned == 1).all()


def test_zero_state_offsets_follow_the_interleaved_rule():
    cfg = config_from_descriptor("d12")
    P, r = 4, 2
    plan = zero.ZeroPlan(cfg, P, r, 1)
    lay = cfg.layout()
    seg = next(s for s in plan.segments if s.tensor == "qkvw" and s.layer == 5)
    slot = lay["qkvw"]
    assert seg.length == slot.size // P
    assert seg.param_off == slot.offset + 5 * slot.size + r * (slot.size // P)
    assert seg.state_off == slot.offset // P + 5 * (slot.size // P)


def test_zero_validation_errors():
    with pytest.raises(zero.ZeroError):
        zero.validate_zero_stage(4)
    cfg = config_from_descriptor("d12")
    assert zero.validate_sharding(cfg, 7, 1)  # 768 is not divisible by 7
    assert not zero.validate_sharding(cfg, 7, 0)
    with pytest.raises(zero.ZeroError):
        zero.ZeroPlan(cfg, 7, 0, 2)


# ------------------------------------------------------------------------------------- flags / dry run
def test_flag_parser_defaults_and_values():
    a = flags_mod.parse_flags([], "gpt2")
    assert (a.B, a.T, a.max_steps, a.learning_rate, a.zero_stage, a.recompute, a.use_master_weights) == (4, 1024, -1, 3e-4, 0, 1, 1)
    a = flags_mod.parse_flags("-e d12 -b 64 -t 1024 -d 524288 -r 0 -z 1 -c 0.1 -l 6e-4 -q 0 -u 700 -nk 5 -nm 100 -sl 5.0 -pi fs -pf /tmp/x".split(), "gpt2")
    assert (a.load_filename, a.B, a.total_batch_size, a.zero_stage, a.weight_decay, a.warmup_iterations) == ("d12", 64, 524288, 1, 0.1, 700)
    assert (a.checkpoints_keep, a.major_checkpoint_every, a.skip_update_lossz, a.nccl_init_method, a.fs_path) == (5, 100, 5.0, "fs", "/tmp/x")
    l = flags_mod.parse_flags([], "llama3")
    assert (l.load_filename, l.T, l.max_steps) == ("llama3:1B", 2048, 0)
    for bad in (["-e"], ["e", "d12"], ["-zz", "1"], ["-b", "x"], ["-ge", "1"]):
        with pytest.raises(flags_mod.FlagError):
            flags_mod.parse_flags(bad, "llama3")
    flags_mod.parse_flags(["-ge", "1"], "gpt2")


def test_dry_runs(capsys, tmp_path):
    assert train_mod.run("-e d12 -x 0 -z 1 -pn 8".split(), "gpt2") == 0
    out = capsys.readouterr().out
    assert "GPT dry run: max_seq_len=1024 vocab=50257 padded_vocab=50304 layers=12 heads=12" in out
    assert "parameters=124475904" in out and "ZeRO-1 layout validated for 8 process(es)." in out
    assert train_mod.run("-e llama3:8B -z 3 -pn 8".split(), "llama3") == 0
    assert "Llama dry run: ZeRO-3 layout validated for 8 process(es)." in capsys.readouterr().out
    assert train_mod.run("-e d12 -x 0 -z 4".split(), "gpt2") == 1
    assert train_mod.run("-e d12 -x 0 -z 1 -pn 7".split(), "gpt2") == 1
    assert train_mod.run("-e d12 -x 0 -t 2048".split(), "gpt2") == 1
    assert train_mod.run("-e d12 -x 0 -pn 2 -pr 2".split(), "gpt2") == 1
    # from a checkpoint header (tiny model) and a corrupted payload
    cfg = ModelConfig(family="gpt2", max_seq_len=64, vocab_size=100, padded_vocab_size=128, num_layers=1, num_heads=2,
                      num_kv_heads=2, channels=64, hidden_dim=256)
    path = str(tmp_path / "m.bin")
    formats.write_model(path, cfg, torch.zeros(cfg.num_parameters(), dtype=torch.bfloat16))
    assert train_mod.run(["-e", path, "-x", "0", "-t", "64"], "gpt2") == 0
    with open(path, "ab") as f:
        f.write(b"xx")
    assert train_mod.run(["-e", path, "-x", "0", "-t", "64"], "gpt2") == 1


# ------------------------------------------------------------------------------------- formats
def test_model_file_round_trip_and_golden_header(tmp_path):
    cfg = ModelConfig(family="gpt2", max_seq_len=64, vocab_size=100, padded_vocab_size=128, num_layers=2, num_heads=2,
                      num_kv_heads=2, channels=64, hidden_dim=256)
    params = torch.randn(cfg.num_parameters()).to(torch.bfloat16)
    path = str(tmp_path / "model_00000010.bin")
    formats.write_model(path, cfg, params)
    h = formats.read_header(path)
    assert list(h[:8]) == [20240326, 5, 64, 100, 2, 2, 64, 128]
    assert os.path.getsize(path) == 1024 + 2 * cfg.num_parameters()
    cfg2, p2 = formats.read_model(path)
    assert cfg2.num_parameters() == cfg.num_parameters() and torch.equal(p2, params)
    # raw payload is exactly the tensor order of the layout
    raw = np.fromfile(path, dtype=np.uint16, offset=1024)
    assert np.array_equal(raw, params.view(torch.int16).numpy().view(np.uint16))
    lcfg = ModelConfig(family="llama3", max_seq_len=128, vocab_size=256, padded_vocab_size=256, num_layers=1, num_heads=4,
                       num_kv_heads=2, channels=64, hidden_dim=192, tied_embeddings=False, use_scaled_rope=True)
    lp = str(tmp_path / "l.bin")
    formats.write_model(lp, lcfg, torch.zeros(lcfg.num_parameters(), dtype=torch.bfloat16))
    h = formats.read_header(lp)
    assert list(h[:9]) == [20240803, 5, 128, 256, 1, 4, 2, 64, 192] and h[11] == 500000 and h[12] == 1
    c3, _ = formats.read_model(lp)
    assert c3.family == "llama3" and c3.num_kv_heads == 2 and c3.use_scaled_rope and not c3.tied_embeddings
    with pytest.raises(formats.FormatError):
        bad = str(tmp_path / "bad.bin")
        open(bad, "wb").write(np.zeros(256, dtype=np.int32).tobytes())
        formats.read_model(bad)


def test_state_file_round_trip(tmp_path):
    n = 1000
    m, v, master = torch.randn(n), torch.rand(n), torch.randn(n)
    path = str(tmp_path / "state_00000005_00001.bin")
    blob = b"\x01\x02\x03" * 10
    formats.write_state(path, "gpt2", 2, 1, 5, m, v, master, 0x1234567890ABCDEF, 42, 3, 77, blob)
    raw = open(path, "rb").read()
    h = np.frombuffer(raw[:1024], dtype=np.int32)
    assert list(h[:6]) == [20240527, 1, 2, 1, 1, 1] and h[10] == 5
    assert struct.unpack_from("<Q", raw, 80)[0] == 0x1234567890ABCDEF and struct.unpack_from("<Q", raw, 120)[0] == 3
    assert len(raw) == 1024 + 3 * n * 4 + len(blob)
    m2, v2, ma2 = torch.zeros(n), torch.zeros(n), torch.zeros(n)
    info = formats.read_state(path, "gpt2", 2, 1, m2, v2, ma2)
    assert torch.equal(m, m2) and torch.equal(v, v2) and torch.equal(master, ma2)
    assert (info["step"], info["rng_state"], info["rng_state_last_update"], info["shard_idx"], info["sample_idx"]) == (5, 0x1234567890ABCDEF, 42, 3, 77)
    assert info["shuffle_blob"] == blob
    with pytest.raises(formats.FormatError):
        formats.read_state(path, "gpt2", 4, 1, m2, v2, ma2)  # different world size
    with pytest.raises(formats.FormatError):
        formats.read_state(path, "llama3", 2, 1, m2, v2, ma2)


def test_find_max_step(tmp_path):
    assert formats.find_max_step(str(tmp_path)) == -1
    for s in (10, 200, 30):
        open(tmp_path / ("DONE_%08d" % s), "w").close()
    assert formats.find_max_step(str(tmp_path)) == 200
    assert formats.checkpoint_paths("o", 7, 3) == ("o/model_00000007.bin", "o/state_00000007_00003.bin", "o/DONE_00000007")


# ------------------------------------------------------------------------------------- loaders
def _write_shards(tmp_path, n_shards, ntok, desc="gpt-2", prefix="train"):
    rng = np.random.default_rng(0)
    all_toks = []
    for i in range(n_shards):
        toks = rng.integers(0, 50000 if desc == "gpt-2" else 120000, size=ntok)
        formats.write_tokens(str(tmp_path / f"{prefix}_{i:03d}.bin"), toks, desc)
        all_toks.append(toks)
    return all_toks


@pytest.mark.parametrize("desc", ["gpt-2", "llama-3"])
def test_dataloader_sequential(tmp_path, desc):
    B, T, P = 2, 8, 2
    shards = _write_shards(tmp_path, 2, 100, desc)
    loaders = [DataLoader(str(tmp_path / "train_*.bin"), B, T, r, P, False) for r in range(P)]
    assert loaders[0].num_tokens == 200 and loaders[0].num_shards == 2
    per_shard = (100 - 1) // (B * T * P)
    for shard in (0, 1, 0):  # wraps around after the last shard
        for s in range(per_shard):
            for r, ld in enumerate(loaders):
                x, y = ld.next_batch()
                off = s * B * T * P + r * B * T
                assert np.array_equal(x.numpy().ravel(), shards[shard][off: off + B * T])
                assert np.array_equal(y.numpy().ravel(), shards[shard][off + 1: off + B * T + 1])
    assert formats.read_tokens(str(tmp_path / "train_000.bin")).dtype == (np.uint16 if desc == "gpt-2" else np.uint32)


def test_dataloader_shuffle_resume_is_exact(tmp_path):
    B, T = 2, 8
    _write_shards(tmp_path, 3, 200)
    a = DataLoader(str(tmp_path / "train_*.bin"), B, T, 0, 1, True)
    seq = [a.next_batch()[0].clone() for _ in range(20)]
    b = DataLoader(str(tmp_path / "train_*.bin"), B, T, 0, 1, True)
    for i in range(7):
        b.next_batch()
    state = (b.current_shard_idx, b.current_sample_idx, b.shuffle_state())
    assert len(state[2]) > 2520
    c = DataLoader(str(tmp_path / "train_*.bin"), B, T, 0, 1, True)
    c.resume(*state)
    for i in range(7, 20):
        assert torch.equal(c.next_batch()[0], seq[i])
    # shuffling permutes samples (not a prefix of the sequential order) but covers one epoch exactly
    d = DataLoader(str(tmp_path / "train_*.bin"), B, T, 0, 1, False)
    seq_plain = [d.next_batch()[0].clone() for _ in range(20)]
    assert any(not torch.equal(x, y) for x, y in zip(seq, seq_plain))
    # ring of pinned buffers: a batch stays valid while the next one is produced
    e = DataLoader(str(tmp_path / "train_*.bin"), B, T, 0, 1, False, ring=3)
    x0 = e.next_batch()[0]
    keep = x0.clone()
    e.next_batch()
    e.next_batch()
    assert torch.equal(x0, keep)


def test_dataloader_errors(tmp_path):
    from llm_kittens_b200.utils.hostlib import HostError

    with pytest.raises(HostError):
        DataLoader(str(tmp_path / "nothing_*.bin"), 2, 8)
    bad = tmp_path / "bad.bin"
    hdr = np.zeros(256, dtype=np.int32)
    hdr[0], hdr[1], hdr[2] = 20240520, 1, 50
    bad.write_bytes(hdr.tobytes() + b"\0" * 10)
    with pytest.raises(HostError):
        DataLoader(str(bad), 2, 8)
    _write_shards(tmp_path, 1, 10)
    with pytest.raises(HostError):
        DataLoader(str(tmp_path / "train_*.bin"), 2, 8)  # shard smaller than one batch


def test_evalloader_and_stat_losses(tmp_path):
    B, T = 8, 32
    examples = []
    rng = np.random.default_rng(1)
    for i in range(5):
        ctx = rng.integers(0, 1000, size=5 + i).tolist()
        ends = [rng.integers(0, 1000, size=3 + j).tolist() for j in range(4)]
        examples.append({"label": i % 4, "ctx_tokens": ctx, "ending_tokens": ends})
    path = str(tmp_path / "eval.bin")
    formats.write_evalfile(path, examples)
    ld = EvalLoader(path, B, T, 0, 1)
    assert ld.num_examples == 5 and ld.num_batches == 3
    seen = 0
    for bi in range(ld.num_batches):
        x, y = ld.next_batch()
        for slot in range(B // 4):
            if seen >= 5:
                assert ld.label[slot].item() == -1
                continue
            ex = examples[seen]
            assert ld.label[slot].item() == ex["label"]
            for c in range(4):
                row = slot * 4 + c
                n_ctx, end = len(ex["ctx_tokens"]), ex["ending_tokens"][c]
                assert x[row, :n_ctx].tolist() == ex["ctx_tokens"]
                assert x[row, n_ctx:n_ctx + len(end)].tolist() == end
                assert y[row, n_ctx - 1:n_ctx - 1 + len(end)].tolist() == end
                assert ld.mask[row].sum().item() == len(end) and ld.mask[row, n_ctx - 1].item() == 1
            seen += 1
        # losses that make the labelled completion the best one
        losses = np.ones((B, T), dtype=np.float32)
        for slot in range(B // 4):
            lab = ld.label[slot].item()
            if lab >= 0:
                losses[slot * 4 + lab] = 0.1
        expected = sum(1 for s in range(B // 4) if ld.label[s].item() >= 0)
        assert ld.stat_losses(losses) == expected
    # two processes split the examples
    l0, l1 = EvalLoader(path, B, T, 0, 2), EvalLoader(path, B, T, 1, 2)
    l0.next_batch()
    l1.next_batch()
    assert l0.label[0].item() == examples[0]["label"] and l1.label[0].item() == examples[3]["label"]


def test_tokenizer_round_trip(tmp_path):
    toks = [b"hello", b" world", b"\n", b"\xf0\x9f", b"\x01"]
    path = str(tmp_path / "tok.bin")
    formats.write_tokenizer(path, toks, eot_token=3)
    t = Tokenizer(path)
    assert t.init_ok and t.vocab_size == 5 and t.eot_token == 3
    assert [t.decode(i) for i in range(5)] == toks and t.decode(99) is None
    assert Tokenizer.safe_text(t.decode(4)) == "" and Tokenizer.safe_text(t.decode(0)) == "hello"
    assert not Tokenizer(str(tmp_path / "missing.bin")).init_ok


# ------------------------------------------------------------------------------------- small host utilities
def test_schedulers():
    s = LearningRateScheduler("cosine", 6e-4, 700, 20000, 0.0)
    assert abs(s.get(0) - 6e-4 / 700) < 1e-10 and abs(s.get(699) - 6e-4) < 1e-9
    assert abs(s.get(700) - 6e-4) < 1e-9 and s.get(20000) < 1e-9
    mid = s.get(700 + (20000 - 700) // 2)
    assert abs(mid - 3e-4) < 2e-6
    lin = LearningRateScheduler("linear", 1.0, 0, 100, 0.1)
    assert abs(lin.get(50) - 0.55) < 1e-6 and abs(lin.get(100) - 0.1) < 1e-6
    assert LearningRateScheduler("constant", 0.5, 10, 100, 0.0).get(3) == 0.5
    w = LearningRateScheduler("wsd", 1.0, 10, 100, 0.0)
    assert abs(w.get(4) - 0.5) < 1e-6 and w.get(50) == 1.0 and w.get(79) == 1.0
    assert abs(w.get(85) - (1 - math.sqrt(0.25))) < 1e-6
    with pytest.raises(ValueError):
        LearningRateScheduler("exp", 1.0, 0, 10, 0.0)


def test_logger_and_validators(tmp_path):
    lg = Logger(str(tmp_path), 0, resume=False)
    lg.log_val(0, 10.9876543)
    for s in range(5):
        lg.log_train(s, 10.0 - s, 6e-4, 1.2345)
    lg.log_eval(4, 0.25)
    text = open(tmp_path / "main.log").read().splitlines()
    assert text[0] == "s:0 tel:10.9877" and text[1] == "s:0 trl:10.0000 lr:0.000600 norm:1.23" and text[-1] == "s:4 eval:0.2500"
    Logger(str(tmp_path), 1, resume=False).log_train(0, 1, 1, 1)  # other ranks do not write
    assert len(open(tmp_path / "main.log").read().splitlines()) == 7
    Logger(str(tmp_path), 0, resume=True).log_train(5, 4.5, 6e-4, 1.0)  # resume appends
    parsed = parse_log(str(tmp_path / "main.log"))
    assert parsed["train"][5][0] == 4.5 and parsed["val"][0] == 10.9877 and parsed["eval"][4] == 0.25
    assert validate_log(str(tmp_path / "main.log"), final_step=5, max_final_train_loss=5.0) == []
    assert validate_log(str(tmp_path / "main.log"), final_step=9) != []
    other = tmp_path / "b"
    lb = Logger(str(other), 0)
    for s in range(6):
        lb.log_train(s, 10.0 - s + (0.5 if s == 3 else 0.01), 6e-4, 1.0)
    probs = compare_logs(str(tmp_path / "main.log"), str(other / "main.log"), rel_tol=0.01, abs_tol=0.02)
    assert len(probs) >= 1 and any("step 3" in p for p in probs)
    Logger(str(tmp_path), 0, resume=False)  # fresh start wipes the file
    assert open(tmp_path / "main.log").read() == ""


def test_outlier_detector():
    d = OutlierDetector()
    rng = np.random.default_rng(0)
    vals = rng.normal(5.0, 1.0, size=128)
    for v in vals:
        assert math.isnan(d.update(v))
    z = d.update(5.0 + 6.0)
    window = np.concatenate([vals[1:], [11.0]])
    assert abs(z - (11.0 - window.mean()) / window.std()) < 1e-9
    c = OutlierDetector()
    for _ in range(128):
        c.update(1.0)
    assert c.update(1.0) == 0.0


def test_rng_matches_torch_and_state_round_trip():
    g = Mt19937(42)
    torch.manual_seed(42)
    assert np.abs(torch.rand(1000).numpy() - g.uniform_(1000)).max() == 0.0
    a = torch.normal(0.0, 0.02, (4099,)).numpy()
    b = g.normal_(4099, 0.0, 0.02)
    assert np.abs(a - b).max() < 1e-7  # same stream and transform; libm differences of an ulp
    h = Mt19937(7)
    h.randint32()
    blob = h.state()
    assert len(blob) == 2520
    nxt = [h.randint32() for _ in range(700)]
    h2 = Mt19937(1)
    h2.set_state(blob)
    assert [h2.randint32() for _ in range(700)] == nxt
    # MT19937 reference value: seed 5489, first output
    assert Mt19937(5489).randint32() == 3499211612
    p = Mt19937(3).permutation(50)
    assert sorted(p.tolist()) == list(range(50))
    x = Xorshift(1337)
    u = [x.u32() for _ in range(3)]
    y = Xorshift(1337)
    assert [y.u32() for _ in range(3)] == u and 0.0 <= Xorshift(5).f32() < 1.0
    logits = np.array([0.0, 10.0, 0.0], dtype=np.float32)
    assert sample_softmax(logits, 0.5) == 1 and sample_softmax(logits, 0.0) == 0 and sample_softmax(logits, 0.99999) == 2


def test_check_cli_zero_layout_log_and_checkpoint(tmp_path, capsys):
    """The run-validation commands (reference: dev/validate_zero_layout.py, dev/validate_training_log.py,
    dev/compare_training_logs.py, dev/validate_llama_checkpoint_artifacts.py)."""
    from llm_kittens_b200.cli import check

    assert check.main(["zero-layout", "--models", "d12", "llama3.2:1B", "gpt3:c768", "--world", "1", "2", "4", "8"]) == 0
    log = Logger(str(tmp_path), 0)
    for s, l in enumerate([5.0, 4.0, 3.5]):
        log.log_train(s, l, 1e-3, 1.0)
    main_log = str(tmp_path / "main.log")
    assert check.main(["log", main_log, "--final-step", "2", "--max-train-loss", "4.0"]) == 0
    assert check.main(["log", main_log, "--final-step", "7"]) == 1
    assert check.main(["compare", main_log, main_log]) == 0
    # checkpoint directory: a model file of the right size, one state file, DONE marker
    cfg = ModelConfig(family="gpt2", max_seq_len=64, vocab_size=100, padded_vocab_size=128, num_layers=1, num_heads=2,
                      num_kv_heads=2, channels=64, hidden_dim=256)
    n = cfg.num_parameters()
    params = torch.zeros(n, dtype=torch.bfloat16)
    model_path, state_path, done_path = formats.checkpoint_paths(str(tmp_path), 4, 0)
    formats.write_model(model_path, cfg, params)
    z = torch.zeros(n, dtype=torch.float32)
    formats.write_state(state_path, cfg.family, 1, 0, 4, z, z, None, 1, 2, 0, 0, b"")
    assert check.main(["checkpoint", str(tmp_path)]) == 1          # no DONE marker yet
    open(done_path, "w").close()
    assert check.main(["checkpoint", str(tmp_path)]) == 0
    with open(model_path, "ab") as f:
        f.write(b"\0\0")
    assert check.main(["checkpoint", str(tmp_path), "--step", "4"]) == 1
    capsys.readouterr()


def test_native_scheduler_outlier_and_logger_match_the_python_versions(tmp_path):
    """The C++ host library's schedules, outlier detector and logger against their Python restatements."""
    import math
    import random

    from llm_kittens_b200.utils.outlier import NativeOutlierDetector, OutlierDetector
    from llm_kittens_b200.utils.schedulers import LearningRateScheduler

    for kind in LearningRateScheduler.TYPES:
        s = LearningRateScheduler(kind, 6e-4, 70, 1000, 0.1)
        assert s._native is not None
        for step in list(range(0, 1001, 7)) + [69, 70, 71, 799, 800, 801, 1000]:
            a, b = s.get(step), s.get_python(step)
            assert abs(a - b) <= 2e-7 * max(abs(b), 1e-6) + 1e-10, (kind, step, a, b)
    with pytest.raises(ValueError):
        LearningRateScheduler("cosine", 1e-3, 10, 100, 0.0).get(101)
    rnd_ = random.Random(0)
    nat, py = NativeOutlierDetector(), OutlierDetector()
    for i in range(400):
        v = rnd_.gauss(3.0, 0.5) + (8.0 if i == 300 else 0.0)
        za, zb = nat.update(v), py.update(v)
        assert (math.isnan(za) and math.isnan(zb)) or abs(za - zb) < 1e-9
        if i == 300:
            assert za > 5.0
    a_dir, b_dir = tmp_path / "native", tmp_path / "python"
    for d, native in ((a_dir, True), (b_dir, False)):
        lg = Logger(str(d), 0, native=native)
        assert (lg._h is not None) == native
        lg.log_val(0, 10.98765)
        for st in range(3):
            lg.log_train(st, 10.0 - st * 0.333333, 6e-4 * (st + 1) / 3, 1.2345 + st)
        lg.log_eval(2, 0.2512)
        Logger(str(d), 0, resume=True, native=native).log_train(3, 1.5, 1e-4, 0.5)
    assert open(a_dir / "main.log", "rb").read() == open(b_dir / "main.log", "rb").read()


def test_grouped_gemm_wrapper_falls_back_to_one_launch_per_group(monkeypatch):
    """Shape logic of ops/gemm.py on CPU tensors with the native call replaced by a recorder: rows that are not a
    multiple of the tile height (or, for NN / TN, a K that is not a multiple of 64) must turn a grouped call into one
    plain call per group on the right row slices; eligible shapes make ONE grouped call."""
    from llm_kittens_b200.ops import _native, gemm

    calls = []
    monkeypatch.setattr(_native, "require_cuda_tensor", lambda *a, **k: None)
    monkeypatch.setattr(_native, "status_word", lambda: None)
    monkeypatch.setattr(_native, "call", lambda name, *a: calls.append((name, a)))
    monkeypatch.setattr(gemm, "tile_rows", lambda: 256)

    class FakeLib:
        @staticmethod
        def llmk_gemm_workspace_bytes(*a):
            return 0

    monkeypatch.setattr(_native, "lib", lambda: FakeLib)
    bf = torch.bfloat16
    G, M, N, K = 3, 512, 384, 128
    a, w, bias = torch.zeros(G * M, K, dtype=bf), torch.zeros(G, N, K, dtype=bf), torch.zeros(G, N, dtype=bf)
    out = gemm.gemm_nt(a, w, bias=bias, groups=G)
    assert out.shape == (G * M, N) and len(calls) == 1 and calls[0][0] == "llmk_gemm_grouped"
    assert calls[0][1][8:12] == (M, N, K, G)
    calls.clear()
    M2 = 200                                            # not a multiple of the tile height: three plain calls
    a2 = torch.arange(G * M2 * K, dtype=torch.float32).reshape(G * M2, K).to(bf)
    out2 = torch.zeros(G * M2, N, dtype=bf)
    gemm.gemm_nt(a2, w, bias=bias, out=out2, groups=G)
    assert [c[0] for c in calls] == ["llmk_gemm"] * G
    for g, (_, args) in enumerate(calls):
        A, B, C, bias_g = args[2], args[3], args[4], args[6]
        assert A.data_ptr() == a2[g * M2:].data_ptr() and A.shape == (M2, K)
        assert B.data_ptr() == w[g].data_ptr() and B.shape == (N, K)
        assert C.data_ptr() == out2[g * M2:].data_ptr() and bias_g.data_ptr() == bias[g].data_ptr()
        assert args[8:11] == (M2, N, K)
    calls.clear()
    # TN with K (tokens per group) not a multiple of 64: per-group calls on token slices, outputs [G, M, N]
    Kt = 100
    dy, x = torch.zeros(G * Kt, 256, dtype=bf), torch.zeros(G * Kt, N, dtype=bf)
    gw = torch.zeros(G, 256, N, dtype=bf)
    gemm.gemm_tn(dy, x, out=gw, accumulate=True, groups=G)
    assert [c[0] for c in calls] == ["llmk_gemm"] * G
    for g, (_, args) in enumerate(calls):
        assert args[2].data_ptr() == dy[g * Kt:].data_ptr() and args[3].data_ptr() == x[g * Kt:].data_ptr()
        assert args[4].data_ptr() == gw[g].data_ptr() and args[7].data_ptr() == gw[g].data_ptr()
        assert args[8:11] == (256, N, Kt)


def test_debug_state_commands_round_trip(tmp_path):
    """`check write-debug-state` + `check debug-state` on a small model file: the PyTorch path reproduces the stored
    logits, loss and gradients; a perturbed model file is reported tensor by tensor."""
    import torch

    from llm_kittens_b200.cli import check
    from llm_kittens_b200.models.config import ModelConfig
    from llm_kittens_b200.oracle.torch_model import TorchTransformer
    from llm_kittens_b200.utils import formats

    cfg = ModelConfig(family="gpt2", max_seq_len=64, vocab_size=300, padded_vocab_size=320, num_layers=2, num_heads=2,
                      num_kv_heads=2, channels=64, hidden_dim=256)
    model = TorchTransformer(cfg, device="cpu", dtype=torch.float32)
    model.init_weights(7)
    mp, sp = str(tmp_path / "model.bin"), str(tmp_path / "debug_state.bin")
    formats.write_model(mp, cfg, model.params)
    assert check.main(["write-debug-state", mp, sp, "--batch", "2", "--seq", "32"]) == 0
    state = formats.read_debug_state(sp, cfg.vocab_size, model.num_parameters)
    assert state["x"].shape == (2, 32) and state["logits"].shape == (2, 32, 300) and state["grads"].shape == (model.num_parameters,)
    # the model file stores bf16 unless asked otherwise: compare through the same file
    assert check.check_debug_state(mp, sp, device="cpu") == []
    model.params[model.layout["fcw"].offset: model.layout["fcw"].offset + 50].add_(0.5)
    formats.write_model(str(tmp_path / "other.bin"), cfg, model.params)
    problems = check.check_debug_state(str(tmp_path / "other.bin"), sp, device="cpu")
    assert problems and any("logits" in p or "gradient" in p for p in problems)


def test_device_preflight_against_a_stand_in_machine(capsys):
    """`check device` on pretended machines: eight B200s pass, a Hopper card or a missing peer link is named, a machine
    without GPUs fails (the job of the reference's dev/cuda/cuda_runtime_check.cu:53-133 for this framework's target)."""
    from llm_kittens_b200.cli import check

    class Probe:
        def __init__(self, devs, no_peer=(), pairs=74):
            self.devs, self.no_peer, self.pairs, self.touched = devs, set(no_peer), pairs, []

        def versions(self):
            return "580.159", "12.8"

        def devices(self):
            return self.devs

        def can_access_peer(self, a, b):
            return (a, b) not in self.no_peer

        def touch(self, dev):
            self.touched.append(dev)

        def pair_clusters(self, dev):
            return self.pairs

    b200 = {"name": "NVIDIA B200", "major": 10, "minor": 0, "sms": 148, "memory": 183359 << 20}
    h100 = {"name": "NVIDIA H100", "major": 9, "minor": 0, "sms": 132, "memory": 80 << 30}
    lines = []
    p = Probe([b200] * 8)
    assert check.check_device(peers=True, probe=p, out=lines.append) == [] and p.touched == list(range(8))
    assert any("sm_100" in l and "148 SMs" in l for l in lines) and any("74 resident CTA pairs" in l for l in lines)
    bad = check.check_device(probe=Probe([b200, h100]), out=lines.append)
    assert len(bad) == 1 and "device 1" in bad[0] and "sm_90" in bad[0]
    bad = check.check_device(peers=True, probe=Probe([b200] * 2, no_peer=[(0, 1)]), out=lines.append)
    assert len(bad) == 1 and "from device 0 to device 1" in bad[0]
    assert check.check_device(probe=Probe([b200], pairs=0), out=lines.append)
    assert check.check_device(probe=Probe([]), out=lines.append) == ["no CUDA devices visible to the runtime"]
    if not torch.cuda.is_available():
        assert check.main(["device"]) == 1 and "no CUDA devices" in capsys.readouterr().out


def test_sampling_hands_the_training_buffers_back_untouched():
    """``generate`` re-runs the model on (1, T) windows; afterwards the training-shape activations AND the token /
    target buffers must be the very tensors they were (a captured CUDA graph of the micro-step keeps their addresses)."""
    from types import SimpleNamespace

    from llm_kittens_b200.runtime.sampling import generate

    class Stub:
        def __init__(self):
            self.config = SimpleNamespace(max_seq_len=128, vocab_size=50)
            self.device = "cpu"
            self.B, self.T = 4, 128
            self.acts = {"marker": torch.zeros(1)}
            self.tokens = torch.zeros(4, 128, dtype=torch.int32)
            self.targets = torch.zeros(4, 128, dtype=torch.int32)
            self.calls = []

        def forward(self, x, y):
            B, T = x.shape
            if self.acts is None or (self.B, self.T) != (B, T):    # what Transformer.allocate does for a new shape
                self.B, self.T, self.acts = B, T, {"marker": torch.ones(1)}
                self.tokens = torch.zeros(B, T, dtype=torch.int32)
                self.targets = torch.zeros(B, T, dtype=torch.int32)
            self.tokens.copy_(x)
            self.calls.append((B, T))

        def logits_view(self):
            g = torch.Generator().manual_seed(len(self.calls))
            return torch.randn(self.B, self.T, 64, generator=g)

    m = Stub()
    acts, tokens, targets = m.acts, m.tokens, m.targets
    out = generate(m, [7], 70)
    assert len(out) == 70 and out[0] == 7 and all(0 <= t < 50 for t in out)
    assert m.calls[0] == (1, 64) and m.calls[-1] == (1, 128)            # windows padded to multiples of 64
    assert (m.B, m.T) == (4, 128) and m.acts is acts and m.tokens is tokens and m.targets is targets
    assert int(tokens.abs().sum()) == 0                                  # the training buffers were not written
    m.calls.clear()
    assert generate(m, [7], 70) == out                                   # same logits, same coin stream, same sample


def test_dataloader_properties_over_random_geometries(tmp_path_factory):
    """Random shard counts and sizes (unequal shards), batch shapes and rank counts: in sequential mode every rank reads
    exactly the windows that the reference's loader formula gives (llmc/dataloader.h:174-218: per shard
    (tokens - 1) // (B*T*P) samples, rank r at offset sample*B*T*P + r*B*T, next shard afterwards, wrapping around); in
    shuffle mode one epoch hands out every (shard, sample) window of a rank exactly once and targets are inputs
    shifted by one token."""
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st

    @settings(max_examples=25, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
    @given(sizes=st.lists(st.integers(40, 400), min_size=1, max_size=4), B=st.integers(1, 3), T=st.integers(2, 9),
           P=st.integers(1, 3), seed=st.integers(0, 1000))
    def run(sizes, B, T, P, seed):
        chunk = B * T * P
        if min(sizes) - 1 < chunk:
            return
        d = tmp_path_factory.mktemp("geo")
        rng = np.random.default_rng(seed)
        shards = []
        for i, n in enumerate(sizes):
            toks = rng.integers(0, 60000, size=n)
            formats.write_tokens(str(d / f"s_{i:03d}.bin"), toks, "gpt-2")
            shards.append(toks)
        per_shard = [(n - 1) // chunk for n in sizes]
        for r in range(P):
            ld = DataLoader(str(d / "s_*.bin"), B, T, r, P, False)
            assert ld.num_tokens == sum(sizes) and ld.num_shards == len(sizes)
            for shard in list(range(len(sizes))) + [0]:                       # one epoch and the wrap-around
                for s in range(per_shard[shard]):
                    x, y = ld.next_batch()
                    off = s * chunk + r * B * T
                    assert np.array_equal(x.numpy().ravel(), shards[shard][off: off + B * T]), (sizes, B, T, P, r, shard, s)
                    assert np.array_equal(y.numpy().ravel(), shards[shard][off + 1: off + B * T + 1])
            ld.close()
        # shuffle: an epoch is a permutation of the rank's windows
        r = P - 1
        ld = DataLoader(str(d / "s_*.bin"), B, T, r, P, True)
        want = {(shard, s) for shard in range(len(sizes)) for s in range(per_shard[shard])}
        index = {}
        for shard in range(len(sizes)):
            for s in range(per_shard[shard]):
                off = s * chunk + r * B * T
                index.setdefault(tuple(shards[shard][off: off + B * T + 1]), set()).add((shard, s))
        seen = []
        for _ in range(len(want)):
            x, y = ld.next_batch()
            xs, ys = x.numpy().ravel(), y.numpy().ravel()
            assert np.array_equal(xs[1:], ys[:-1])
            key = tuple(list(xs) + [ys[-1]])
            assert key in index
            seen.append(key)
        # every window handed out belongs to the rank; windows with unique contents appear exactly once
        from collections import Counter
        counts = Counter(seen)
        for key, c in counts.items():
            assert c <= len(index[key])
        assert sum(counts.values()) == len(want)
        ld.close()

    run()


def test_file_formats_round_trip_over_random_models_and_states(tmp_path_factory):
    """Random small model geometries of all three families through write_model / read_model (bit-exact parameters, equal
    configuration), random optimizer states through write_state / read_state, random token shards and evaluation
    files through their writers and the native readers."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    fam = st.sampled_from(["gpt2", "llama3", "moe"])

    @settings(max_examples=20, deadline=None)
    @given(family=fam, layers=st.integers(1, 3), heads=st.sampled_from([1, 2, 4]), kv_div=st.sampled_from([1, 2]),
           head_size=st.sampled_from([64, 128]), hidden_mul=st.sampled_from([2, 4]), vocab=st.integers(50, 300), seed=st.integers(0, 10**6),
           world=st.sampled_from([1, 2, 4]))
    def run(family, layers, heads, kv_div, head_size, hidden_mul, vocab, seed, world):
        d = tmp_path_factory.mktemp("fmt")
        C = heads * head_size
        kv = max(1, heads // kv_div) if family == "llama3" else heads
        extra = dict(num_experts=4, top_k=2) if family == "moe" else {}
        # what the llm.c headers can express: GPT-2 / MoE files imply hidden = 4 C, Llama files have no padded vocabulary
        if family == "llama3":
            vocab = (vocab + 63) // 64 * 64
            padded, hidden = vocab, hidden_mul * C
        else:
            padded, hidden = (vocab + 127) // 128 * 128, 4 * C
        cfg = ModelConfig(family=family, max_seq_len=64, vocab_size=vocab, padded_vocab_size=padded, num_layers=layers,
                          num_heads=heads, num_kv_heads=kv, channels=C, hidden_dim=hidden, **extra)
        g = torch.Generator().manual_seed(seed)
        n = cfg.layout().total
        params = torch.randn(n, generator=g).to(torch.bfloat16)
        path = str(d / "model.bin")
        formats.write_model(path, cfg, params)
        cfg2, back = formats.read_model(path)
        assert torch.equal(back.view(torch.int16), params.view(torch.int16))
        for f in ("family", "max_seq_len", "vocab_size", "padded_vocab_size", "num_layers", "num_heads", "num_kv_heads", "channels",
                  "hidden_dim"):
            assert getattr(cfg2, f) == getattr(cfg, f), f
        if family == "moe":
            assert (cfg2.num_experts, cfg2.top_k) == (4, 2)
        assert os.path.getsize(path) == 1024 + 2 * n           # 256-int header + bf16 payload, nothing else
        # optimizer state of one rank
        shard = max(8, (n // world) // 8 * 8)
        m, v, master = (torch.randn(shard, generator=g) for _ in range(3))
        rank = seed % world
        spath = str(d / "state.bin")
        blob = bytes(range(7)) * 3
        formats.write_state(spath, family, world, rank, 17, m, v, master, 123456789, 987654321, 2, 5, blob)
        m2, v2, ma2 = torch.zeros(shard), torch.zeros(shard), torch.zeros(shard)
        info = formats.read_state(spath, family, world, rank, m2, v2, ma2)
        assert torch.equal(m2, m) and torch.equal(v2, v) and torch.equal(ma2, master)
        assert (info["step"], info["rng_state"], info["rng_state_last_update"], info["shard_idx"], info["sample_idx"]) == (17, 123456789, 987654321, 2, 5)
        assert info["shuffle_blob"] == blob
        with pytest.raises(formats.FormatError):
            formats.read_state(spath, family, world, (rank + 1) % world if world > 1 else 1, m2, v2, ma2)

    run()


def test_model_header_refuses_geometries_the_file_cannot_express():
    odd = ModelConfig(family="gpt2", max_seq_len=64, vocab_size=100, padded_vocab_size=128, num_layers=1, num_heads=1, num_kv_heads=1,
                      channels=64, hidden_dim=128)
    with pytest.raises(formats.FormatError):
        formats.model_header(odd)
    odd = ModelConfig(family="llama3", max_seq_len=64, vocab_size=100, padded_vocab_size=128, num_layers=1, num_heads=1, num_kv_heads=1,
                      channels=64, hidden_dim=128)
    with pytest.raises(formats.FormatError):
        formats.model_header(odd)


def test_process_layout_from_torchrun_mpirun_and_flags():
    """Job size, rank and device index: from torch.distributed.run's environment, from Open MPI's (the reference's
    binaries are started by mpirun and ask MPI), or from the -pn / -pr / -pg flags (one task per GPU under srun)."""
    a = flags_mod.parse_flags([], "gpt2")                           # defaults: -pi mpi, -pn 1
    assert train_mod.resolve_processes(a, {}) == (1, 0, "mpi", 0)
    assert train_mod.resolve_processes(a, {"WORLD_SIZE": "8", "RANK": "5", "LOCAL_RANK": "5"}) == (8, 5, "env", 5)
    ompi = {"OMPI_COMM_WORLD_SIZE": "16", "OMPI_COMM_WORLD_RANK": "11", "OMPI_COMM_WORLD_LOCAL_RANK": "3"}
    assert train_mod.resolve_processes(a, ompi) == (16, 11, "mpi", 3)
    del ompi["OMPI_COMM_WORLD_LOCAL_RANK"]
    assert train_mod.resolve_processes(a, ompi) == (16, 11, "mpi", 3)       # 11 % 8 GPUs per node
    b = flags_mod.parse_flags(["-pn", "16", "-pr", "9", "-pg", "4", "-pi", "tcp", "-ps", "10.0.0.1"], "gpt2")
    assert train_mod.resolve_processes(b, {}) == (16, 9, "tcp", 1)
    assert train_mod.resolve_processes(b, ompi) == (16, 9, "tcp", 1)         # explicit flags win over MPI's environment with -pi tcp
    # torchrun's environment is not used for an explicit tcp / fs rendezvous either
    assert train_mod.resolve_processes(b, {"WORLD_SIZE": "2", "RANK": "1"}) == (16, 9, "tcp", 1)


def test_zero_plans_over_random_geometries_including_experts():
    """Random model geometries (all three families) and rank counts: whenever ``validate_sharding`` accepts a pair, the
    ranks' segments tile the parameter buffer exactly once (dense tensors in P equal parts per layer, every expert with
    one owner), state offsets stay inside the rank's state buffer without overlap, and every shard is a whole number
    of 16-byte units (what the vectorised optimizer kernels assume)."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    @settings(max_examples=60, deadline=None)
    @given(family=st.sampled_from(["gpt2", "llama3", "moe"]), layers=st.integers(1, 4), heads=st.sampled_from([1, 2, 3, 4, 6, 8]),
           head_size=st.sampled_from([64, 128]), vocab_blocks=st.integers(1, 6), P=st.sampled_from([1, 2, 3, 4, 6, 8]),
           experts=st.sampled_from([2, 4, 8]), stage=st.sampled_from([1, 2, 3]))
    def run(family, layers, heads, head_size, vocab_blocks, P, experts, stage):
        C = heads * head_size
        V = vocab_blocks * 128
        extra = dict(num_experts=experts, top_k=2) if family == "moe" else {}
        cfg = ModelConfig(family=family, max_seq_len=64, vocab_size=V, padded_vocab_size=V, num_layers=layers, num_heads=heads,
                          num_kv_heads=heads, channels=C, hidden_dim=4 * C, **extra)
        if family == "moe" and P > 1 and experts % P and P % experts:
            return                                   # experts neither split over the ranks nor ranks over the experts
        if zero.validate_sharding(cfg, P, stage):
            with pytest.raises(zero.ZeroError):
                zero.ZeroPlan(cfg, P, 0, stage)
            return
        lay = cfg.layout()
        owned = np.zeros(lay.total, dtype=np.int16)
        for r in range(P):
            plan = zero.ZeroPlan(cfg, P, r, stage)
            used = np.zeros(plan.state_elements, dtype=np.int8)
            for s in plan.segments:
                assert s.length > 0 and s.length % 8 == 0 and s.param_off % 8 == 0 and s.state_off % 8 == 0, (s, P)
                owned[s.param_off: s.param_off + s.length] += 1
                used[s.state_off: s.state_off + s.length] += 1
            assert used.max() <= 1, "two segments of one rank share optimizer state"
            rows = plan.segment_rows()
            assert sum(n for _, _, _, n, _ in rows) == sum(s.length for s in plan.segments)
        if family == "moe" and P > experts:
            # more ranks than experts: an expert has one owner, the other ranks of its group hold no state for it
            assert owned.max() == 1
            dense = np.ones(lay.total, dtype=bool)
            for slot in lay.slots:
                if slot.spec.expert:
                    dense[slot.offset: slot.offset + slot.total] = False
            assert (owned[dense] == 1).all()
        else:
            assert (owned == 1).all(), (family, P, int((owned != 1).sum()))

    run()


@pytest.mark.parametrize("family", ["gpt2", "llama3", "moe"])
def test_sampling_on_the_pytorch_models_leaves_a_training_step_unchanged(family):
    """``generate`` between two training steps of the PyTorch reference models (the surface the CUDA models share): the
    step after sampling gives the same loss as without sampling, and the sample is reproducible."""
    from llm_kittens_b200.oracle.torch_model import TorchTransformer
    from llm_kittens_b200.runtime.sampling import generate
    from llm_kittens_b200.runtime.trainer import Trainer

    extra = dict(num_experts=4, top_k=2) if family == "moe" else {}
    V = 256
    cfg = ModelConfig(family=family, max_seq_len=128, vocab_size=V, padded_vocab_size=V, num_layers=2, num_heads=2, num_kv_heads=2,
                      channels=64, hidden_dim=256, **extra)
    g = torch.Generator().manual_seed(5)
    batches = [(torch.randint(0, V, (2, 64), generator=g, dtype=torch.int32), torch.randint(0, V, (2, 64), generator=g, dtype=torch.int32))
               for _ in range(3)]

    def run(sample: bool):
        model = TorchTransformer(cfg, device="cpu", dtype=torch.float32)
        model.init_weights(42)
        tr = Trainer(model, learning_rate=1e-3)
        losses, text = [], None
        for i, b in enumerate(batches):
            losses.append(tr.train_step([b]).loss)
            if sample and i == 0:
                acts = model.acts
                text = generate(model, [0], 70)
                assert model.acts is acts and (model.B, model.T) == (2, 64)
                assert generate(model, [0], 70) == text
        return losses, text

    plain, _ = run(False)
    sampled, text = run(True)
    assert sampled == plain
    assert len(text) == 70 and all(0 <= t < V for t in text)
