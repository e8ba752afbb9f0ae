"""Whole-model checks of the CUDA path against the PyTorch fp32 oracle with the same parameters:
loss, logits, every gradient tensor (per-tensor tolerance ``thr + 0.079*|ref|`` in the spirit of the
reference's test_gpt2.cu:9-50), multi-step loss parity (tolerance 0.05 like test_gpt2.cu:326-347),
recompute levels agreeing with each other, and determinism."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def small_gpt2(L=2, C=256, NH=4, T=128, V=1000, Vp=1024):
    from llm_kittens_b200.models.config import ModelConfig

    return ModelConfig(family="gpt2", max_seq_len=T, vocab_size=V, padded_vocab_size=Vp, num_layers=L, num_heads=NH,
                       num_kv_heads=NH, channels=C, hidden_dim=4 * C)


def small_llama(L=2, C=256, NH=4, NKVH=2, T=128, V=1024, H=768, tied=False):
    from llm_kittens_b200.models.config import ModelConfig

    return ModelConfig(family="llama3", max_seq_len=T, vocab_size=V, padded_vocab_size=V, num_layers=L, num_heads=NH,
                       num_kv_heads=NKVH, channels=C, hidden_dim=H, tied_embeddings=tied)


def batch(cfg, B, T, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, cfg.vocab_size, (B, T), generator=g, dtype=torch.int32)
    y = torch.randint(0, cfg.vocab_size, (B, T), generator=g, dtype=torch.int32)
    return x, y


def make_pair(cfg, recompute=0):
    from llm_kittens_b200.models.transformer import Transformer
    from llm_kittens_b200.oracle.torch_model import TorchTransformer

    model = Transformer(cfg, device="cuda", recompute=recompute)
    model.init_weights(42)
    # make biases / norm weights non-trivial so their gradients are exercised
    torch.manual_seed(1)
    for slot in model.layout.slots:
        if slot.spec.init in ("zeros", "ones"):
            seg = model.params[slot.offset: slot.offset + slot.total]
            seg.add_((torch.randn(seg.numel(), device="cuda") * 0.05).to(seg.dtype))
    oracle = TorchTransformer(cfg, device="cuda", dtype=torch.float32)
    oracle.load_parameters(model.params.float())
    return model, oracle


@pytest.mark.parametrize("family", ["gpt2", "llama3", "llama3_tied"])
def test_loss_logits_grads_match_oracle(family):
    cfg = small_gpt2() if family == "gpt2" else small_llama(tied=(family == "llama3_tied"))
    model, oracle = make_pair(cfg)
    x, y = batch(cfg, 4, 128)
    for m in (model, oracle):
        m.zero_grad()
        m.forward(x.cuda(), y.cuda())
    assert abs(model.mean_loss() - oracle.mean_loss()) < 0.02
    # logits were overwritten by dlogits in the CUDA path: compare a no-grad forward
    model.forward(x.cuda(), y.cuda(), compute_dlogits=False)
    lg = model.logits_view()[..., : cfg.vocab_size].float()
    assert (lg - oracle.logits_view()[..., : cfg.vocab_size]).abs().max().item() < 0.1
    model.forward(x.cuda(), y.cuda())
    model.backward()
    oracle.backward()
    from llm_kittens_b200.ops import _native

    _native.check_status()
    for slot in model.layout.slots:
        got = model.grads[slot.offset: slot.offset + slot.total].float()
        ref = oracle.grads[slot.offset: slot.offset + slot.total]
        tol = 2e-3 + 0.079 * ref.abs()
        bad = ((got - ref).abs() > tol)
        frac = bad.float().mean().item()
        assert frac < 2e-3, f"{slot.spec.name}: {frac:.4%} of gradient entries outside tolerance; max err {(got - ref).abs().max().item()}"


@pytest.mark.parametrize("family", ["gpt2", "llama3"])
def test_ten_step_loss_parity(family):
    from llm_kittens_b200.runtime.trainer import Trainer

    cfg = small_gpt2() if family == "gpt2" else small_llama()
    model, oracle = make_pair(cfg)
    tr_n = Trainer(model, learning_rate=1e-3, weight_decay=0.1, use_master_weights=True)
    tr_o = Trainer(oracle, learning_rate=1e-3, weight_decay=0.1)
    x, y = batch(cfg, 4, 128)
    for step in range(10):
        a = tr_n.train_step([(x.pin_memory(), y.pin_memory())])
        b = tr_o.train_step([(x, y)])
        assert abs(a.loss - b.loss) < 0.05, (step, a.loss, b.loss)
        assert abs(a.grad_norm - b.grad_norm) < 0.05 * max(1.0, b.grad_norm), (step, a.grad_norm, b.grad_norm)
    assert a.loss < 0.8 * tr_o.model.config.vocab_size  # sanity
    assert b.loss < 6.0


def test_gpt2_124m_ten_step_loss_parity_full_size(capsys):
    """The reference's whole-model gate at full size (test_gpt2.cu:257-347): GPT-2 124M (12 layers, 768 channels,
    vocabulary 50257 padded to 50304), B=4, T=64, token ids uniform from seed 1337, the same batch for ten AdamW
    steps at lr 1e-4, random init N(0, 0.02) with scaled residual projections; the bf16 CUDA path against the fp32
    PyTorch model with the same initial parameters, per-step loss within 0.05."""
    from llm_kittens_b200.models.config import config_from_descriptor
    from llm_kittens_b200.models.transformer import Transformer
    from llm_kittens_b200.oracle.torch_model import TorchTransformer
    from llm_kittens_b200.runtime.trainer import Trainer

    cfg = config_from_descriptor("d12")
    assert (cfg.num_layers, cfg.channels, cfg.num_heads, cfg.vocab_size, cfg.padded_vocab_size) == (12, 768, 12, 50257, 50304)
    model = Transformer(cfg, device="cuda", recompute=0)
    model.init_weights(42)
    oracle = TorchTransformer(cfg, device="cuda", dtype=torch.float32)
    oracle.load_parameters(model.params.float())
    g = torch.Generator().manual_seed(1337)
    x = torch.randint(0, cfg.vocab_size, (4, 64), generator=g, dtype=torch.int32)
    y = torch.randint(0, cfg.vocab_size, (4, 64), generator=g, dtype=torch.int32)
    tr_n = Trainer(model, learning_rate=1e-4, weight_decay=0.0, use_master_weights=True)
    tr_o = Trainer(oracle, learning_rate=1e-4, weight_decay=0.0)
    ours, ref = [], []
    for step in range(10):
        a = tr_n.train_step([(x.pin_memory(), y.pin_memory())])
        b = tr_o.train_step([(x, y)])
        ours.append(a.loss)
        ref.append(b.loss)
        assert abs(a.loss - b.loss) < 0.05, (step, a.loss, b.loss)
        assert abs(a.grad_norm - b.grad_norm) < 0.05 * max(1.0, b.grad_norm), (step, a.grad_norm, b.grad_norm)
    assert ref[-1] < ref[0] - 1.0   # ten steps on one batch: the loss falls by more than one nat
    with capsys.disabled():
        print("\nGPT-2 124M B=4 T=64 ten-step losses, CUDA bf16:", [round(v, 4) for v in ours])
        print("GPT-2 124M B=4 T=64 ten-step losses, fp32 oracle:", [round(v, 4) for v in ref])


@pytest.mark.parametrize("family", ["gpt2", "llama3"])
def test_recompute_levels_agree_and_are_deterministic(family):
    cfg = small_gpt2() if family == "gpt2" else small_llama()
    x, y = batch(cfg, 2, 128)
    grads = []
    for r in (0, 1, 2, 3, 0):
        model, _ = make_pair(cfg, recompute=r)
        model.zero_grad()
        model.forward(x.cuda(), y.cuda())
        model.backward()
        grads.append(model.grads.clone())
    for gr in grads[1:]:
        assert torch.equal(grads[0], gr)


def test_grad_accumulation_matches_big_batch():
    cfg = small_gpt2()
    model, _ = make_pair(cfg)
    x, y = batch(cfg, 4, 128)
    model.zero_grad()
    model.forward(x.cuda(), y.cuda())
    model.backward()
    full, loss_full = model.grads.float().clone(), model.mean_loss()
    model.zero_grad()
    for i in range(2):
        model.forward(x[2 * i: 2 * i + 2].cuda(), y[2 * i: 2 * i + 2].cuda(), grad_accum_steps=2, micro_step=i)
        model.backward(last_micro_step=(i == 1))
    assert abs(model.mean_loss() - loss_full) < 2e-3
    err = (model.grads.float() - full).abs()
    assert (err > 2e-3 + 0.05 * full.abs()).float().mean().item() < 2e-3


def small_moe(L=2, C=256, NH=4, T=128, V=1000, Vp=1024, E=8, K=2, capacity_factor=1.25):
    from llm_kittens_b200.models.config import ModelConfig

    return ModelConfig(family="moe", max_seq_len=T, vocab_size=V, padded_vocab_size=Vp, num_layers=L, num_heads=NH,
                       num_kv_heads=NH, channels=C, hidden_dim=4 * C, num_experts=E, top_k=K, capacity_factor=capacity_factor,
                       aux_loss_coef=0.01)


def test_moe_ops_against_torch():
    """Router, deterministic slot assignment with capacity dropping, dispatch / combine round trip."""
    from llm_kittens_b200.ops import moe as moe_ops

    N, C, E, K, cap = 512, 256, 8, 2, 96
    x = (torch.randn(N, C, device="cuda")).to(torch.bfloat16)
    wr = (torch.randn(E, C, device="cuda") * 0.1).to(torch.bfloat16)
    probs, idx, w = moe_ops.router_fwd(x, wr, K)
    ref_p = torch.softmax(x.float() @ wr.float().T, -1)
    assert (probs - ref_p).abs().max().item() < 1e-4
    tp, ti = ref_p.topk(K, -1)
    assert torch.equal(idx.long(), ti)
    assert (w - tp / tp.sum(-1, keepdim=True)).abs().max().item() < 1e-4
    slot, counts = moe_ops.assign_slots(idx, E, cap)
    onehot = torch.nn.functional.one_hot(ti.reshape(-1), E)
    ref_slot = (onehot.cumsum(0) - 1)[torch.arange(N * K, device="cuda"), ti.reshape(-1)]
    ref_slot = torch.where(ref_slot < cap, ref_slot, torch.full_like(ref_slot, -1)).view(N, K)
    assert torch.equal(slot.long(), ref_slot)
    assert torch.equal(counts.long(), onehot.sum(0).clamp(max=cap))
    assert (slot < 0).any()  # the capacity is tight enough to drop something
    recv = torch.full((E * cap, C), 7.0, device="cuda", dtype=torch.bfloat16)
    moe_ops.dispatch(moe_ops.ptr_table([recv]), x, idx, slot, w, counts, E, cap)
    back = torch.zeros(E * cap, C, device="cuda", dtype=torch.bfloat16)
    moe_ops.return_rows(moe_ops.ptr_table([back]), recv, C, E, cap)
    # identity experts: combine must give sum_k w_k x for kept assignments, padded slots are zero
    out = torch.zeros(N, C, device="cuda", dtype=torch.bfloat16)
    moe_ops.combine(out, None, back, idx, slot, w, cap)
    keep = (slot >= 0).float()
    ref = (w * keep).sum(-1, keepdim=True) * x.float()
    assert (out.float() - ref).abs().max().item() < 0.03
    for e in range(E):
        pad = back[e * cap + counts[e].item(): (e + 1) * cap]
        assert pad.numel() == 0 or pad.abs().max().item() == 0


@pytest.mark.parametrize("E,cf,way_back", [(8, 1.25, "pull"), (6, 1.25, "pull"), (8, 2.0, "pull"), (8, 2.0, "scatter"), (8, 1.25, "push")])
def test_moe_model_matches_oracle(E, cf, way_back, monkeypatch):
    """E = 6 is not a multiple of 8: the router's gradient GEMMs run on a zero-padded router matrix. Capacity factor 2
    makes every expert's row block a whole number of GEMM tiles (256 rows), which is when the second GEMM stores its
    rows straight into the senders' buffers from its epilogue instead of through the return kernel. The three ways
    back (the combine pulls its rows from the owners; the GEMM's epilogue scatters them; a return kernel pushes them) must
    all match."""
    monkeypatch.setenv("LLMK_MOE_RETURN", way_back)
    monkeypatch.setenv("LLMK_MOE_DISPATCH", "pull" if way_back == "pull" else "push")   # all-pull, and the two push designs
    from llm_kittens_b200.models.moe import MoETransformer
    from llm_kittens_b200.oracle.torch_model import TorchTransformer
    from llm_kittens_b200.ops import _native

    cfg = small_moe(E=E, capacity_factor=cf)
    model = MoETransformer(cfg, device="cuda", recompute=0)
    model.init_weights(42)
    torch.manual_seed(1)
    for slot in model.layout.slots:
        if slot.spec.init in ("zeros", "ones"):
            seg = model.params[slot.offset: slot.offset + slot.total]
            seg.add_((torch.randn(seg.numel(), device="cuda") * 0.05).to(seg.dtype))
    rw = model.layout["routerw"]
    model.params[rw.offset: rw.offset + rw.total].mul_(20.0)   # make routing decisive (no near-ties)
    oracle = TorchTransformer(cfg, device="cuda", dtype=torch.float32)
    oracle.load_parameters(model.params.float())
    x, y = batch(cfg, 4, 128)
    model.zero_grad()
    model.forward(x.cuda(), y.cuda())
    model.backward()
    # the oracle follows the routing choices of the CUDA path (weights, drops and gradients are its own)
    oracle.forced_routing = [model.acts["top_idx"][l].clone() for l in range(cfg.num_layers)]
    oracle.zero_grad()
    oracle.forward(x.cuda(), y.cuda())
    oracle.backward()
    _native.check_status()
    assert abs(model.mean_loss() - oracle.mean_loss()) < 0.02
    assert abs(model.aux_loss() - float(oracle.acts["aux_acc"].item())) < 2e-3
    for slot in model.layout.slots:
        got = model.grads[slot.offset: slot.offset + slot.total].float()
        ref = oracle.grads[slot.offset: slot.offset + slot.total]
        bad = ((got - ref).abs() > 5e-3 + 0.1 * ref.abs()).float().mean().item()
        assert bad < 0.03, f"{slot.spec.name}: {bad:.3%} of gradient entries outside tolerance"
    # a few optimizer steps reduce the loss
    from llm_kittens_b200.runtime.trainer import Trainer

    tr = Trainer(model, learning_rate=1e-3)
    l0 = tr.train_step([(x.pin_memory(), y.pin_memory())]).loss
    for _ in range(5):
        l1 = tr.train_step([(x.pin_memory(), y.pin_memory())]).loss
    assert l1 < l0


def test_cuda_graph_micro_step_matches_eager():
    """The captured forward+backward replays the same kernels: losses and parameters are bit-identical."""
    from llm_kittens_b200.models.config import ModelConfig
    from llm_kittens_b200.models.transformer import Transformer
    from llm_kittens_b200.ops import _native
    from llm_kittens_b200.runtime.trainer import Trainer

    cfg = ModelConfig(family="gpt2", max_seq_len=128, vocab_size=512, padded_vocab_size=512, num_layers=2, num_heads=2,
                      num_kv_heads=2, channels=128, hidden_dim=512)
    g = torch.Generator().manual_seed(5)
    data = [[(torch.randint(0, 512, (4, 128), generator=g, dtype=torch.int32).pin_memory(),
              torch.randint(0, 512, (4, 128), generator=g, dtype=torch.int32).pin_memory()) for _ in range(2)] for _ in range(5)]
    results = []
    for use_graph in (False, True):
        model = Transformer(cfg, device="cuda", recompute=1)
        model.init_weights(7)
        tr = Trainer(model, learning_rate=1e-3, weight_decay=0.1)
        tr.enable_cuda_graph(use_graph)
        losses = [tr.train_step(step).loss for step in data]
        _native.check_status()
        assert (tr._graph is not None) == use_graph
        results.append((losses, model.params.clone()))
    assert results[0][0] == results[1][0]
    assert torch.equal(results[0][1], results[1][1])


def test_validation_loop_without_syncs_reads_every_batch_intact(tmp_path):
    """A loop that queues forwards faster than the GPU runs them (d12-size model, two pinned ring slots, no sync
    between batches) must see the same tokens as a loop that syncs after every batch: the loader may not refill a
    pinned buffer whose upload has not run yet."""
    from llm_kittens_b200.data import prepare
    from llm_kittens_b200.models.config import config_from_descriptor
    from llm_kittens_b200.models.transformer import Transformer
    from llm_kittens_b200.utils.dataloader import DataLoader

    B, T, nb = 16, 1024, 8
    prepare.prepare_synthetic(str(tmp_path / "data"), 200_000, vocab_size=50257, seed=5)
    pattern = str(tmp_path / "data" / "synthetic_train_*.bin")
    cfg = config_from_descriptor("d12")
    model = Transformer(cfg, device="cuda", recompute=0)
    model.init_weights(42)

    def run(sync_every_batch):
        loader = DataLoader(pattern, B, T, 0, 1, should_shuffle=False, ring=2)
        per_batch = torch.zeros(nb, device="cuda")
        for i in range(nb):
            x, y = loader.next_batch()
            model.forward(x, y, compute_dlogits=False)
            per_batch[i:i + 1].copy_(model.acts["loss_acc"])
            if sync_every_batch:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        loader.close()
        return per_batch.cpu()

    safe = run(True)
    fast = run(False)
    assert torch.equal(safe, fast), (safe, fast)
    assert len(set(safe.tolist())) == nb    # the batches differ, so a duplicated batch would have shown


def test_non_finite_gradient_skips_the_update_on_the_gpu():
    """An inf written into a gradient on the host side of the step: the AdamW kernel reads the zero clip scale and
    leaves master weights, moments and parameters as they were; the step is reported as skipped."""
    from llm_kittens_b200.models.transformer import Transformer
    from llm_kittens_b200.runtime.trainer import Trainer

    cfg = small_gpt2()
    model = Transformer(cfg, device="cuda", recompute=0)
    model.init_weights(42)
    tr = Trainer(model, learning_rate=1e-3, weight_decay=0.1)
    x, y = batch(cfg, 4, 128)
    tr.train_step([(x.cuda(), y.cuda())])
    before, m_before, master_before = model.params.clone(), tr.m.clone(), tr.master.clone()
    tr.accumulate([(x.cuda(), y.cuda())])
    model.grads[7:8].fill_(float("inf"))
    tr.update(1e-3)
    loss, norm, bad = tr.read_scalars()
    assert bad
    assert torch.equal(model.params, before) and torch.equal(tr.m, m_before) and torch.equal(tr.master, master_before)
    r = tr.train_step([(x.cuda(), y.cuda())])
    assert not r.skipped and torch.isfinite(model.params.float()).all()


def test_debug_state_gate_on_the_cuda_path(tmp_path):
    """The exported-artefact gate: a model file and the fp32 debug state written from it by the PyTorch model are
    checked against the CUDA path (logits, loss, every gradient tensor)."""
    from llm_kittens_b200.cli import check
    from llm_kittens_b200.oracle.torch_model import TorchTransformer
    from llm_kittens_b200.utils import formats

    cfg = small_gpt2()
    ref = TorchTransformer(cfg, device="cpu", dtype=torch.float32)
    ref.init_weights(11)
    mp, sp = str(tmp_path / "model.bin"), str(tmp_path / "debug_state.bin")
    formats.write_model(mp, cfg, ref.params)
    check.write_debug_state(mp, sp, B=4, T=128)
    assert check.check_debug_state(mp, sp, device="cuda") == []
