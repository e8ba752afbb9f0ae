"""Each CUDA op against a plain PyTorch fp32 reference of the same op. Tolerances follow the
reference's kernel smoke tests (LayerNorm out 0.08 / stats 0.05 / grads 0.12: dev/cuda/test_layernorm.cu:325-327;
RMSNorm 0.04 / 0.01: test_rmsnorm.cu:229-230; RoPE 0.02: test_rope.cu:150; attention fwd 0.08 /
bwd 0.20: test_attention.cu:355-356) and are mostly much tighter here."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def rnd(*shape, scale=1.0, dtype=BF):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def maxerr(a, b):
    return (a.float() - b.float()).abs().max().item()


@pytest.mark.parametrize("N,C", [(64, 768), (1000, 768), (3, 1024), (257, 2048), (128, 4096), (33, 1600)])
def test_layernorm_fwd_bwd(N, C):
    from llm_kittens_b200.ops import norm

    x, w, b = rnd(N, C), rnd(C, scale=0.5) + 1, rnd(C, scale=0.1)
    out, mean, rstd = norm.layernorm_fwd(x, w, b)
    xf = x.float().requires_grad_(True)
    wf, bf_ = w.float().requires_grad_(True), b.float().requires_grad_(True)
    ref = torch.nn.functional.layer_norm(xf, (C,), wf, bf_, 1e-5)
    assert maxerr(out, ref) < 0.04
    assert maxerr(mean, x.float().mean(-1)) < 1e-3
    assert maxerr(rstd, 1 / torch.sqrt(x.float().var(-1, unbiased=False) + 1e-5)) < 1e-2
    dout = rnd(N, C)
    ref.backward(dout.float())
    dinp0 = rnd(N, C)
    dinp = dinp0.clone()
    dw, db = torch.zeros(C, device="cuda", dtype=BF), torch.zeros(C, device="cuda", dtype=BF)
    norm.layernorm_bwd(dinp, dw, db, dout, x, w, mean, rstd, accumulate_dinp=True)
    assert maxerr(dinp, xf.grad + dinp0.float()) < 0.06
    assert maxerr(dw, wf.grad) < 0.02 * max(1.0, wf.grad.abs().max().item())
    assert maxerr(db, bf_.grad) < 0.02 * max(1.0, bf_.grad.abs().max().item())
    # deterministic
    dw2, db2, dinp2 = torch.zeros_like(dw), torch.zeros_like(db), dinp0.clone()
    norm.layernorm_bwd(dinp2, dw2, db2, dout, x, w, mean, rstd, accumulate_dinp=True)
    assert torch.equal(dw, dw2) and torch.equal(db, db2) and torch.equal(dinp, dinp2)


def test_residual_layernorm():
    from llm_kittens_b200.ops import norm

    N, C = 300, 768
    a, b, w, bias = rnd(N, C), rnd(N, C), rnd(C) + 1, rnd(C)
    res, out, mean, rstd = norm.residual_layernorm_fwd(a, b, w, bias)
    r = (a.float() + b.float()).to(BF)
    assert torch.equal(res, r)
    ref = torch.nn.functional.layer_norm(r.float(), (C,), w.float(), bias.float(), 1e-5)
    assert maxerr(out, ref) < 0.04


@pytest.mark.parametrize("N,C", [(64, 2048), (100, 4096), (5, 768)])
def test_rmsnorm(N, C):
    from llm_kittens_b200.ops import norm

    x, w = rnd(N, C), rnd(C, scale=0.3) + 1
    out, rstd = norm.rmsnorm_fwd(x, w, 1e-5)
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    assert maxerr(out, ref) < 0.04
    assert maxerr(rstd, torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)) < 0.01
    dout = rnd(N, C)
    ref.backward(dout.float())
    dinp = torch.zeros(N, C, device="cuda", dtype=BF)
    dw = torch.zeros(C, device="cuda", dtype=BF)
    norm.rmsnorm_bwd(dinp, dw, dout, x, w, rstd, accumulate_dinp=False)
    assert maxerr(dinp, xf.grad) < 0.04
    assert maxerr(dw, wf.grad) < 0.02 * max(1.0, wf.grad.abs().max().item())
    a, b = rnd(N, C), rnd(N, C)
    res, out2, _ = norm.residual_rmsnorm_fwd(a, b, w, 1e-5)
    assert torch.equal(res, (a.float() + b.float()).to(BF))


def test_gelu_swiglu_add():
    from llm_kittens_b200.ops import elementwise as ew

    x = rnd(1000, 3072, scale=2.0)
    xf = x.float().requires_grad_(True)
    ref = torch.nn.functional.gelu(xf, approximate="tanh")
    assert maxerr(ew.gelu_fwd(x), ref) < 0.02
    d = rnd(1000, 3072)
    ref.backward(d.float())
    assert maxerr(ew.gelu_bwd_inplace(d.clone(), x), xf.grad) < 0.03
    g, u, do = rnd(512, 8192), rnd(512, 8192), rnd(512, 8192)
    gf, uf = g.float().requires_grad_(True), u.float().requires_grad_(True)
    r = torch.nn.functional.silu(gf) * uf
    assert maxerr(ew.swiglu_fwd(g, u), r) < 0.07  # |out| reaches ~16 where one bf16 ulp is 0.06
    r.backward(do.float())
    dg, du = ew.swiglu_bwd(do, g, u)
    assert maxerr(dg, gf.grad) < 0.1 and maxerr(du, uf.grad) < 0.1
    ug = torch.cat([u, g], dim=1).contiguous()
    assert torch.equal(ew.swiglu_fused_fwd(ug), ew.swiglu_fwd(g, u))
    dug = ew.swiglu_fused_bwd(do, ug)
    assert torch.equal(dug[:, :8192], du) and torch.equal(dug[:, 8192:], dg)
    a, b = rnd(777, 64), rnd(777, 64)
    assert torch.equal(ew.add(a, b), (a.float() + b.float()).to(BF))


@pytest.mark.parametrize("interleaved", [True, False])
def test_rope(interleaved):
    from llm_kittens_b200.ops import elementwise as ew

    B, T, NH, NKVH, HS = 2, 128, 8, 2, 64
    qkv = rnd(B, T, (NH + 2 * NKVH) * HS)
    freqs = ew.rope_tables(T, HS, 500000.0)
    out = ew.rope_qk_(qkv.clone(), freqs, B, T, NH, NKVH, HS, interleaved=interleaved)
    x = qkv.float().view(B, T, NH + 2 * NKVH, HS)
    cos, sin = freqs[..., 0][None, :, None, :], freqs[..., 1][None, :, None, :]
    ref = x.clone()
    rot = x[:, :, : NH + NKVH]
    if interleaved:
        x0, x1 = rot[..., 0::2], rot[..., 1::2]
        ref[:, :, : NH + NKVH, 0::2] = x0 * cos - x1 * sin
        ref[:, :, : NH + NKVH, 1::2] = x0 * sin + x1 * cos
    else:
        x0, x1 = rot[..., : HS // 2], rot[..., HS // 2:]
        ref[:, :, : NH + NKVH, : HS // 2] = x0 * cos - x1 * sin
        ref[:, :, : NH + NKVH, HS // 2:] = x0 * sin + x1 * cos
    assert maxerr(out, ref.view(B, T, -1)) < 0.02
    back = ew.rope_qk_(out.clone(), freqs, B, T, NH, NKVH, HS, interleaved=interleaved, inverse=True)
    assert maxerr(back, qkv) < 0.05


def test_dbias_and_encoder():
    from llm_kittens_b200.ops import elementwise as ew

    dout = rnd(1000, 2304)
    db0 = rnd(2304)
    db = db0.clone()
    ew.dbias(db, dout, accumulate=True)
    ref_db = db0.float() + dout.float().sum(0)
    assert ((db.float() - ref_db).abs() <= 0.01 * ref_db.abs() + 0.05).all()
    B, T, C, V = 4, 64, 768, 1000
    wte, wpe = rnd(V, C), rnd(T, C)
    tok = torch.randint(0, V, (B, T), device="cuda", dtype=torch.int32)
    tok[0, :10] = 7  # repeated token
    out = ew.encoder_fwd(tok, wte, wpe)
    assert maxerr(out, wte.float()[tok.long()] + wpe.float()[None]) < 0.02
    d = rnd(B, T, C)
    dwte, dwpe = torch.zeros_like(wte), torch.zeros_like(wpe)
    ew.encoder_bwd(dwte, dwpe, d, tok)
    ref_wte = torch.zeros(V, C, device="cuda").index_add_(0, tok.reshape(-1).long(), d.float().view(-1, C))
    assert maxerr(dwte, ref_wte) < 0.06
    assert maxerr(dwpe, d.float().sum(0)) < 0.05
    dwte2, dwpe2 = torch.zeros_like(wte), torch.zeros_like(wpe)
    ew.encoder_bwd(dwte2, dwpe2, d, tok)
    assert torch.equal(dwte, dwte2)


@pytest.mark.parametrize("n,V", [(65536, 50304), (5000, 128256), (2048, 300), (33, 7), (131072, 50304)])
def test_bucket_sort_is_a_stable_sort_by_token(n, V):
    """The device radix sort that buckets positions by token id gives exactly the stable sort (token, position),
    for sizes that are not whole tiles and for vocabularies that need one, two and (hypothetically) more digit passes."""
    from llm_kittens_b200.ops import elementwise as ew

    g = torch.Generator(device="cuda").manual_seed(n)
    tok = torch.randint(0, V, (n,), generator=g, device="cuda", dtype=torch.int32)
    tok[: n // 3] = tok[0]                    # a heavy hitter, as natural text has
    st, sp = ew.bucket_sort(tok, V)
    ref_tok, ref_pos = torch.sort(tok, stable=True)
    assert torch.equal(st, ref_tok) and torch.equal(sp.long(), ref_pos)
    st2, sp2 = ew.bucket_sort(tok, 1 << 20)    # three passes
    assert torch.equal(st2, ref_tok) and torch.equal(sp2.long(), ref_pos)


@pytest.mark.parametrize("rows,V,Vp", [(64, 50257, 50304), (16, 1000, 1024), (8, 128256, 128256)])
def test_fused_classifier(rows, V, Vp):
    from llm_kittens_b200.ops import classifier

    logits = rnd(rows, Vp, scale=2.0)
    tg = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
    lf = logits.float()[:, :V].requires_grad_(True)
    ref_losses = torch.nn.functional.cross_entropy(lf, tg.long(), reduction="none")
    dloss = 1.0 / rows
    (ref_losses.sum() * dloss).backward()
    lg = logits.clone()
    losses = classifier.fused_classifier(lg, tg, V, dloss)
    assert maxerr(losses, ref_losses) < 2e-3
    assert maxerr(lg[:, :V], lf.grad) < 2e-3
    assert lg[:, V:].abs().max().item() == 0 if Vp > V else True
    lg2 = logits.clone()
    l2 = classifier.fused_classifier(lg2, tg, V, dloss, write_dlogits=False)
    assert torch.equal(lg2, logits) and torch.equal(l2, losses)
    tot = torch.zeros(1, device="cuda")
    classifier.sum_scaled(tot, losses, 1.0 / rows)
    assert abs(tot.item() - ref_losses.mean().item()) < 1e-3


def _ref_attention(qkv, B, T, NH, NKVH, HS):
    x = qkv.float().view(B, T, NH + 2 * NKVH, HS)
    q = x[:, :, :NH].transpose(1, 2)
    k = x[:, :, NH:NH + NKVH].transpose(1, 2).repeat_interleave(NH // NKVH, dim=1)
    v = x[:, :, NH + NKVH:].transpose(1, 2).repeat_interleave(NH // NKVH, dim=1)
    s = q @ k.transpose(-1, -2) / math.sqrt(HS)
    mask = torch.ones(T, T, device=qkv.device, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    p = s.softmax(-1)
    o = (p @ v).transpose(1, 2).reshape(B, T, NH * HS)
    return o, torch.logsumexp(s, -1)


@pytest.mark.parametrize("B,T,NH,NKVH,HS", [(2, 128, 4, 4, 64), (1, 256, 12, 12, 64), (2, 192, 8, 2, 64), (1, 128, 4, 2, 128),
                                            (1, 1024, 2, 1, 128)])
def test_attention_fwd_bwd(B, T, NH, NKVH, HS):
    from llm_kittens_b200.ops import _native, attention

    qkv = rnd(B, T, (NH + 2 * NKVH) * HS)
    out_w, lse_w = attention.attention_fwd(qkv, B, T, NH, NKVH, HS, impl="warp")
    out, lse = attention.attention_fwd(qkv, B, T, NH, NKVH, HS, impl="tc")   # tcgen05 path when T % 128 == 0
    _native.check_status()
    assert maxerr(out, out_w) < 0.03 and maxerr(lse, lse_w) < 0.02
    qf = qkv.float().requires_grad_(True)
    ref, ref_lse = _ref_attention(qf, B, T, NH, NKVH, HS)
    assert maxerr(out, ref) < 0.03
    assert maxerr(lse, ref_lse) < 0.02
    dout = rnd(B, T, NH * HS)
    ref.backward(dout.float())
    dqkv_w = attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS, impl="warp")
    assert maxerr(dqkv_w, qf.grad) < 0.08
    dqkv = attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS)
    _native.check_status()
    assert maxerr(dqkv, qf.grad) < 0.08
    dqkv2 = attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS)
    assert torch.equal(dqkv, dqkv2)


@pytest.mark.parametrize("dkv", ["", "1", "2"])
@pytest.mark.parametrize("B,T,NH,NKVH,HS,scale", [(1, 1024, 8, 2, 64, 1.0), (1, 2048, 4, 1, 64, 1.0), (1, 2048, 12, 12, 64, 1.0),
                                                  (1, 4096, 32, 8, 128, 1.0), (1, 1024, 12, 12, 64, 3.0), (1, 2048, 8, 2, 128, 3.0)])
def test_attention_long_sequences(B, T, NH, NKVH, HS, scale, dkv, monkeypatch):
    """The sequence lengths of the training configurations: many key tiles per query tile (the K/V ring wraps
    around), grouped queries long enough for the pipelined dK/dV kernel (chosen by itself for (T/64)*(NH/NKVH) >= 64,
    forced both ways through LLMK_ATTN_BWD_DKV), and inputs scaled so that logits reach +-30 and the row maximum
    jumps by more than 2^8 between key tiles (the lazy rescale of the output accumulator fires)."""
    from llm_kittens_b200.ops import _native, attention

    if dkv:
        monkeypatch.setenv("LLMK_ATTN_BWD_DKV", dkv)
    else:
        monkeypatch.delenv("LLMK_ATTN_BWD_DKV", raising=False)
    torch.manual_seed(T + NH + HS)
    qkv = rnd(B, T, (NH + 2 * NKVH) * HS, scale=scale)
    out, lse = attention.attention_fwd(qkv, B, T, NH, NKVH, HS)
    _native.check_status()
    qf = qkv.float().requires_grad_(True)
    ref, ref_lse = _ref_attention(qf, B, T, NH, NKVH, HS)
    assert maxerr(out, ref) < (0.03 if scale == 1.0 else 0.05 * scale)   # outputs reach |5| at scale 3: one bf16 ulp there is 0.03
    assert maxerr(lse, ref_lse) < 0.02 * max(1.0, scale * scale)
    dout = rnd(B, T, NH * HS)
    ref.backward(dout.float())
    dqkv = attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS)
    _native.check_status()
    assert maxerr(dqkv, qf.grad) < 0.08 * max(1.0, scale * scale)
    dqkv2 = attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS)
    assert torch.equal(dqkv, dqkv2)


def _rope_ref(x, table, B, T, heads, HS, inverse=False):
    """fp32 rotation of the first ``heads`` heads of a packed [B*T, W] tensor, interleaved pairs."""
    x = x.float().clone().view(B, T, -1)
    part = x[..., : heads * HS].reshape(B, T, heads, HS // 2, 2)
    cos, sin = table[..., 0][None, :, None, :], table[..., 1][None, :, None, :]
    if inverse:
        sin = -sin
    x0, x1 = part[..., 0], part[..., 1]
    rot = torch.stack([x0 * cos - x1 * sin, x0 * sin + x1 * cos], dim=-1)
    x[..., : heads * HS] = rot.reshape(B, T, heads * HS)
    return x.view(B * T, -1)


@pytest.mark.parametrize("B,T,NH,NKVH,HS,C", [(2, 128, 4, 2, 64, 256), (1, 256, 8, 2, 128, 512), (1, 1024, 8, 2, 64, 512)])
def test_rope_in_the_qkv_projection_and_in_the_attention_backward(B, T, NH, NKVH, HS, C):
    """RoPE folded into the QKV GEMM's epilogue equals projection followed by an fp32 rotation; the attention backward
    with the table returns dq / dk already rotated back, equal to the plain backward followed by the inverse rotation."""
    from llm_kittens_b200.ops import _native, attention, elementwise as ew, gemm

    torch.manual_seed(B * T + HS)
    W = (NH + 2 * NKVH) * HS
    x, w = rnd(B * T, C), rnd(W, C, scale=0.05)
    table = ew.rope_tables(T, HS, 500000.0, False)
    fused = gemm.gemm_qkv_rope(x, w, table, T, (NH + NKVH) * HS, HS)
    _native.check_status()
    ref = _rope_ref(x.float() @ w.float().T, table, B, T, NH + NKVH, HS)
    assert maxerr(fused, ref) < 0.03
    unfused = ew.rope_qk_(gemm.gemm_nt(x, w), table, B, T, NH, NKVH, HS, interleaved=True)
    assert maxerr(fused, unfused) < 0.05   # the unfused path rounds to bf16 twice
    # backward
    qkv = fused.view(B, T, W)
    out, lse = attention.attention_fwd(qkv, B, T, NH, NKVH, HS)
    dout = rnd(B, T, NH * HS)
    plain = attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS)
    want = _rope_ref(plain.view(B * T, W), table, B, T, NH + NKVH, HS, inverse=True)
    got = attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS, rope=table)
    _native.check_status()
    assert maxerr(got.view(B * T, W), want) < 0.02 * max(1.0, want.abs().max().item())
    assert torch.equal(got.view(B * T, W)[:, (NH + NKVH) * HS:], plain.view(B * T, W)[:, (NH + NKVH) * HS:])   # dv untouched


def test_adamw_and_norm():
    from llm_kittens_b200.ops import optim

    n = 100000
    p32 = torch.randn(n, device="cuda")
    params = p32.to(BF)
    grads = rnd(n, scale=0.1)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    master = torch.empty(n, device="cuda")
    segs, max_len = optim.make_segments([(0, 0, 0, 60000, True), (60000, 60000, 60000, 40000, False)])
    n2 = optim.global_norm2(grads, segs, max_len)
    assert abs(n2.item() - grads.float().pow(2).sum().item()) / n2.item() < 1e-4
    scale, norm_, flag = torch.empty(1, device="cuda"), torch.empty(1, device="cuda"), torch.zeros(1, device="cuda", dtype=torch.int32)
    optim.clip_scale(n2, 1.0, scale, norm_, flag)
    nrm = math.sqrt(n2.item())
    assert abs(scale.item() - min(1.0, 1.0 / nrm)) < 1e-5 and flag.item() == 0
    optim.master_from_params(master, params, segs, max_len)
    assert torch.equal(master, params.float())
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.95, 1e-8, 0.1
    gs = scale.item()
    ref_p = params.float().clone()
    g = grads.float() * gs
    rm = (1 - b1) * g
    rv = (1 - b2) * g * g
    mh, vh = rm / (1 - b1), rv / (1 - b2)
    wdv = torch.cat([torch.full((60000,), wd), torch.zeros(40000)]).cuda()
    ref_p = ref_p - lr * (mh / (vh.sqrt() + eps) + wdv * ref_p)
    optim.adamw(params, master, grads, m, v, segs, max_len, lr, b1, b2, 1, eps, wd, grad_scale_ptr=scale, seed=1234)
    assert maxerr(master, ref_p) < 1e-5
    assert maxerr(m, rm) < 1e-6 and maxerr(v, rv) < 1e-6
    # stochastic rounding: within one bf16 ulp of the fp32 value and unbiased on average
    ulp = (master.abs() * 2 ** -7).clamp_min(1e-30)
    assert ((params.float() - master).abs() <= ulp).all()
    assert abs((params.float() - master).mean().item()) < 1e-4
    p2 = torch.empty_like(params)
    optim.params_from_master(p2, master, segs, max_len, 1234)
    assert torch.equal(p2, params)


def test_scratch_buffers_stay_inside_their_guard_regions():
    """The kernels that write scratch memory through raw pointers (split-K partials, column-sum partials) get
    exactly-sized buffers between canary pages; the canaries must be intact afterwards. The damaged case is made on
    the host (a tensor fill over the whole allocation), not by a kernel."""
    import pytest as _pytest

    from llm_kittens_b200.ops import _native, elementwise as ew, gemm, norm

    _native.set_guards(True)
    try:
        for M, Nn, K in [(768, 768, 4096), (2304, 768, 8192), (520, 264, 1000), (3072, 768, 2048)]:
            a, b = rnd(K, M, scale=0.1), rnd(K, Nn, scale=0.1)
            out = gemm.gemm_tn(a, b)
            assert maxerr(out, a.float().T @ b.float()) < 0.02 * K ** 0.5
        for rows, C in [(1000, 768), (4096, 1024), (777, 2048), (512, 4096)]:
            x, w, bb = rnd(rows, C), rnd(C, scale=0.5) + 1, rnd(C, scale=0.1)
            _, mean, rstd = norm.layernorm_fwd(x, w, bb)
            dinp = torch.zeros(rows, C, device="cuda", dtype=BF)
            dw, db = torch.zeros(C, device="cuda", dtype=BF), torch.zeros(C, device="cuda", dtype=BF)
            norm.layernorm_bwd(dinp, dw, db, rnd(rows, C), x, w, mean, rstd, accumulate_dinp=False)
            _, rstd2 = norm.rmsnorm_fwd(x, w, 1e-5)
            norm.rmsnorm_bwd(dinp, dw, rnd(rows, C), x, w, rstd2, accumulate_dinp=False)
            ew.dbias(db, rnd(rows, C), accumulate=False)
        assert _native.check_guards() >= 8
        _native.check_status()
        # host-made damage is reported
        name, whole, payload = _native._GUARDED[0]
        whole[-1:].fill_(0)
        with _pytest.raises(_native.NativeError, match="guard region"):
            _native.check_guards()
    finally:
        _native.set_guards(False)


def test_peer_flag_wait_runs_out_and_reports_status():
    """Failure detection inside a kernel, without any fault: a wait on a peer flag that nothing sets gives up after its
    limit (0.2 s here), records LLMK_ST_TIMEOUT_PEER with the silent peer's index in the status word and returns; the
    host reads the word and raises; the context stays usable."""
    import time

    import pytest as _pytest

    from llm_kittens_b200.ops import _native, gemm

    lib = _native.lib()
    ctrl = torch.zeros(int(lib.llmk_comm_ctrl_ints()), dtype=torch.int32, device="cuda")
    _native.check_status()
    # every flag of slot 0 already at the awaited epoch: returns at once, status stays clear
    ctrl[:8] = 1
    _native.call("llmk_comm_wait", ctrl, 0, 1, 2, int(2e8), _native.status_word())
    _native.check_status()
    # peer 1 never signals epoch 2
    ctrl[0] = 2
    torch.cuda.synchronize()
    t0 = time.time()
    _native.call("llmk_comm_wait", ctrl, 0, 2, 2, int(2e8), _native.status_word())
    with _pytest.raises(_native.NativeError, match="status 5") as info:
        _native.check_status()
    waited = time.time() - t0
    assert 0.15 < waited < 5.0, waited
    assert "thread=1" in str(info.value)              # the peer that stayed silent
    # the status word was reset by the check and the context still runs kernels
    a, b = rnd(256, 128), rnd(256, 128, scale=0.05)
    assert maxerr(gemm.gemm_nt(a, b), a.float() @ b.float().T) < 0.05
    _native.check_status()
