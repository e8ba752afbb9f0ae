"""tcgen05 GEMM vs an fp32 PyTorch reference (tolerance of the reference's dev/cuda/test_matmul.cu:216
is max-abs 0.5; ours is far tighter because accumulation is fp32 in TMEM)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(torch.bfloat16)


def _close(got, ref, tol):
    err = (got.float() - ref).abs().max().item()
    assert err <= tol, f"max abs err {err} > {tol}"


def _gelu(x):
    return torch.nn.functional.gelu(x, approximate="tanh")


SHAPES_NT = [(128, 256, 64), (256, 512, 128), (384, 768, 768), (200, 264, 72), (1024, 2304, 768), (512, 50304, 768)]


@pytest.mark.parametrize("M,N,K", SHAPES_NT)
def test_gemm_nt_plain_and_bias(M, N, K):
    from llm_kittens_b200.ops import gemm, _native

    a, b, bias = _rand(M, K), _rand(N, K, scale=0.05), _rand(N)
    ref = a.float() @ b.float().T
    _close(gemm.gemm_nt(a, b), ref, 0.05)
    _close(gemm.gemm_nt(a, b, bias=bias), ref + bias.float(), 0.06)
    _native.check_status()


@pytest.mark.parametrize("M,N,K", [(256, 512, 128), (1024, 3072, 768), (200, 264, 72)])
def test_gemm_nt_gelu_and_add(M, N, K):
    from llm_kittens_b200.ops import gemm, _native

    a, b, bias = _rand(M, K), _rand(N, K, scale=0.05), _rand(N)
    ref = a.float() @ b.float().T + bias.float()
    pre = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out = gemm.gemm_nt(a, b, bias=bias, gelu_pre_out=pre)
    _close(pre, ref, 0.06)
    _close(out, _gelu(ref), 0.06)
    res = _rand(M, N)
    out2 = gemm.gemm_nt(a, b, bias=bias, add=res)
    _close(out2, ref + res.float(), 0.08)
    res2 = res.clone()
    gemm.gemm_nt(a, b, bias=bias, add=res2, out=res2)  # in-place residual add
    _close(res2, ref + res.float(), 0.08)
    _native.check_status()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 768, 2304), (1024, 768, 3072), (200, 264, 72), (512, 768, 50304)])
def test_gemm_nn(M, N, K):
    from llm_kittens_b200.ops import gemm, _native

    a, b = _rand(M, K), _rand(K, N, scale=0.05)
    ref = a.float() @ b.float()
    tol = 0.05 if K < 10000 else 0.3
    _close(gemm.gemm_nn(a, b), ref, tol)
    pre = _rand(M, N)
    xg = pre.float().requires_grad_(True)
    _gelu(xg).sum().backward()
    _close(gemm.gemm_nn(a, b, dgelu_of=pre), ref * xg.grad, tol)
    _native.check_status()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (768, 768, 4096), (2304, 768, 8192), (200, 264, 136), (50304, 768, 1024)])
def test_gemm_tn(M, N, K):
    from llm_kittens_b200.ops import gemm, _native

    a, b = _rand(K, M, scale=0.1), _rand(K, N, scale=0.1)
    ref = a.float().T @ b.float()
    out = gemm.gemm_tn(a, b)
    _close(out, ref, 0.1)
    acc = _rand(M, N)
    acc0 = acc.clone()
    gemm.gemm_tn(a, b, out=acc, accumulate=True)
    _close(acc, ref + acc0.float(), 0.15)
    _native.check_status()


@pytest.mark.parametrize("M,N,K", [(768, 768, 4096), (3072, 768, 8192), (3072, 3072, 2048), (200, 136, 1000), (2304, 768, 640)])
def test_gemm_tn_with_bias_gradient_from_the_same_launch(M, N, K):
    """dW and dbias of a linear layer from one kernel: the column sums of dout are taken from the A tiles in shared
    memory. The shapes cover split K (partials finished by the reduction kernel), one split with two tiles per CTA
    pair (sums written by the GEMM kernel itself), a ragged tile and a K that is no multiple of the k-block."""
    from llm_kittens_b200.ops import gemm, _native

    if not gemm.fused_dbias_available():
        pytest.skip("needs the CTA-pair GEMM kernel")
    launches = _native.launch_count()
    a, b = _rand(K, M, scale=0.1), _rand(K, N, scale=0.1)
    ref, ref_db = a.float().T @ b.float(), a.float().sum(0)

    def close_db(got, want):                          # one bf16 rounding of a sum of K values: relative
        err = (got.float() - want).abs()
        bad = err > 0.005 * want.abs() + 0.02
        assert not bad.any(), f"{int(bad.sum())} columns off, worst {err.max().item()}"

    db = torch.full((M,), 7.0, device="cuda", dtype=torch.bfloat16)
    out = gemm.gemm_tn(a, b, dbias=db)
    assert _native.launch_count() == launches + 1     # no stand-alone column-sum kernel ran
    _close(out, ref, 0.1)
    close_db(db, ref_db)
    acc, db2 = _rand(M, N), _rand(M)
    acc0, db0 = acc.clone(), db2.clone()
    gemm.gemm_tn(a, b, out=acc, accumulate=True, dbias=db2)
    _close(acc, ref + acc0.float(), 0.15)
    close_db(db2, ref_db + db0.float())
    # run-to-run bit equality (fixed summation order), and the same bits as the GEMM without the column sums
    db3 = torch.empty_like(db)
    out3 = gemm.gemm_tn(a, b, dbias=db3)
    assert torch.equal(db3, db) and torch.equal(out3, out)
    assert torch.equal(gemm.gemm_tn(a, b), out)
    _native.check_status()


@pytest.mark.parametrize("G,M,N,K", [(4, 512, 512, 256), (2, 256, 1000, 192), (4, 768, 3072, 4096), (2, 200, 264, 128)])
def test_grouped_gemm_tn_with_bias_gradients_per_group(G, M, N, K):
    """The experts of a mixture-of-experts layer: dW [G, M, N] and dbias [G, M] from one grouped launch (the last shape
    has ragged tiles and takes the route of one GEMM per group plus the grouped column-sum kernel)."""
    from llm_kittens_b200.ops import gemm, _native

    if not gemm.fused_dbias_available():
        pytest.skip("needs the CTA-pair GEMM kernel")
    a, b = _rand(G * K, M, scale=0.1), _rand(G * K, N, scale=0.1)
    ref = torch.stack([a[g * K:(g + 1) * K].float().T @ b[g * K:(g + 1) * K].float() for g in range(G)])
    ref_db = torch.stack([a[g * K:(g + 1) * K].float().sum(0) for g in range(G)])
    acc, db = _rand(G, M, N), _rand(G, M)
    acc0, db0 = acc.clone(), db.clone()
    launches = _native.launch_count()
    gemm.gemm_tn(a, b, out=acc, accumulate=True, groups=G, dbias=db)
    if M % 256 == 0 and K % 64 == 0:
        assert _native.launch_count() == launches + 1
    _close(acc, ref + acc0.float(), 0.15)
    err = (db.float() - (ref_db + db0.float())).abs()
    assert not (err > 0.005 * ref_db.abs() + 0.03).any(), err.max().item()
    out, db2 = torch.empty(G, M, N, device="cuda", dtype=torch.bfloat16), torch.empty(G, M, device="cuda", dtype=torch.bfloat16)
    gemm.gemm_tn(a, b, out=out, groups=G, dbias=db2)
    _close(out, ref, 0.1)
    assert not ((db2.float() - ref_db).abs() > 0.005 * ref_db.abs() + 0.02).any()
    assert torch.equal(gemm.gemm_tn(a, b, groups=G).view(G, M, N), out)
    _native.check_status()


@pytest.mark.parametrize("B,T,NH,K", [(2, 256, 4, 256), (4, 1024, 12, 768), (1, 2048, 32, 2048), (3, 128, 3, 192)])
def test_gemm_nn_with_the_attention_backward_row_sums_in_its_epilogue(B, T, NH, K):
    """dO = dres @ W from the GEMM and D[b, h, t] = sum over head h of dO * O from its epilogue, against the stand-alone
    pre-pass of the attention backward and an fp32 formula; the GEMM's own output must not change by a bit."""
    from llm_kittens_b200.ops import attention, gemm, _native

    if not gemm.fused_drow_available(64):
        pytest.skip("entry point not built")
    M, N = B * T, NH * 64
    a, w, o = _rand(M, K), _rand(K, N, scale=0.05), _rand(M, N)
    plain = gemm.gemm_nn(a, w)
    dvec = torch.full((B, NH, T), 7.0, device="cuda", dtype=torch.float32)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    assert gemm.gemm_nn(a, w, out=out, drow_of=(o, dvec, T)) is out
    assert torch.equal(out, plain)
    ref = (plain.float() * o.float()).view(B, T, NH, 64).sum(-1).permute(0, 2, 1)
    assert (dvec - ref).abs().max().item() <= 1e-3 * ref.abs().max().item() + 1e-4
    prep = torch.empty_like(dvec)
    assert attention.attention_bwd_prep(plain, o, prep, B, T, NH, 64)
    assert (dvec - prep).abs().max().item() <= 1e-3 * ref.abs().max().item() + 1e-4
    dvec2 = torch.empty_like(dvec)
    gemm.gemm_nn(a, w, out=out, drow_of=(o, dvec2, T))
    assert torch.equal(dvec2, dvec)
    _native.check_status()


def test_gemm_deterministic():
    from llm_kittens_b200.ops import gemm

    a, b = _rand(4096, 768), _rand(4096, 768)
    o1 = gemm.gemm_tn(a, b).clone()
    o2 = gemm.gemm_tn(a, b)
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("G,M,N,K", [(4, 512, 512, 256), (3, 256, 1000, 192), (2, 200, 264, 128)])
def test_gemm_grouped_matches_per_group_reference(G, M, N, K):
    """One launch for G equal-shaped problems (MoE experts); the last shape has rows that are not a multiple of the
    tile height, which takes the one-launch-per-group path of the wrapper."""
    from llm_kittens_b200.ops import gemm, _native

    # NT with bias + GELU: a [G*M,K], w [G,N,K], bias [G,N]
    a, w, bias = _rand(G * M, K), _rand(G, N, K, scale=0.05), _rand(G, N)
    pre = torch.empty(G * M, N, device="cuda", dtype=torch.bfloat16)
    out = gemm.gemm_nt(a, w, bias=bias, gelu_pre_out=pre, groups=G)
    for g in range(G):
        ref = a[g * M:(g + 1) * M].float() @ w[g].float().T + bias[g].float()
        _close(pre[g * M:(g + 1) * M], ref, 0.06)
        _close(out[g * M:(g + 1) * M], _gelu(ref), 0.06)
    # NN: dy [G*M,N] @ w [G,N,K] -> [G*M,K], with the dGELU factor
    dy = _rand(G * M, N)
    pre2 = _rand(G * M, K)
    dx = gemm.gemm_nn(dy, w, dgelu_of=pre2, groups=G)
    x = pre2.float().requires_grad_(True)
    _gelu(x).sum().backward()
    for g in range(G):
        ref = (dy[g * M:(g + 1) * M].float() @ w[g].float()) * x.grad[g * M:(g + 1) * M]
        _close(dx[g * M:(g + 1) * M], ref, 0.15)
    # TN: per-group weight gradient dy_g^T @ a_g accumulated into [G,N,K]
    dyw = _rand(G * M, N, scale=0.1)
    gw = _rand(G, N, K)
    gw0 = gw.clone()
    gemm.gemm_tn(dyw, a, out=gw, accumulate=True, groups=G)
    for g in range(G):
        ref = gw0[g].float() + dyw[g * M:(g + 1) * M].float().T @ a[g * M:(g + 1) * M].float()
        _close(gw[g], ref, 0.12)
    _native.check_status()


def test_gemm_polls_readiness_flags_of_its_weight_operand():
    """The consumer half of the tile-granular parameter gather: a GEMM whose weight is registered with per-chunk
    flags gives the plain result when the flags carry the expected tick (NT and NN layouts, tiles that span chunk
    borders), and when one chunk's flag never arrives the bounded wait runs out after the given limit: status 5
    (peer flag timeout) is read by the host and the context stays usable."""
    from llm_kittens_b200.ops import _native, gemm

    torch.manual_seed(0)
    M, Nn, K = 512, 640, 256
    a = (torch.randn(M, K, device="cuda") * 0.1).to(torch.bfloat16)
    w = (torch.randn(Nn, K, device="cuda") * 0.1).to(torch.bfloat16)
    d = (torch.randn(M, Nn, device="cuda") * 0.1).to(torch.bfloat16)
    chunk = 10240                       # elements per flag: 40 rows of the weight, so tiles straddle chunks
    nflags = (Nn * K + chunk - 1) // chunk
    flags = torch.zeros(nflags + 3, dtype=torch.int32, device="cuda")
    entry = gemm.register_b_ready(w, flags, 3, chunk, int(0.2e9))
    try:
        plain_nt = gemm.gemm_nt(a, w.clone())
        plain_nn = gemm.gemm_nn(d, w.clone())
        entry[3] = 7
        flags.fill_(7)
        torch.cuda.synchronize()
        assert torch.equal(gemm.gemm_nt(a, w), plain_nt)
        assert torch.equal(gemm.gemm_nn(d, w), plain_nn)
        _native.check_status()
        # an older tick in one flag = a chunk that has not landed: nothing sets it, the wait must run out
        flags[3 + nflags // 2] = 6
        torch.cuda.synchronize()
        gemm.gemm_nt(a, w)
        torch.cuda.synchronize()
        with pytest.raises(_native.NativeError, match="peer flag"):
            _native.check_status()
        flags.fill_(7)
        assert torch.equal(gemm.gemm_nt(a, w), plain_nt)   # the context and the kernels still work
        _native.check_status()
    finally:
        gemm.unregister_b_ready(w)


@pytest.mark.parametrize("M,H,K", [(256, 128, 64), (512, 768, 256), (300, 1024, 200), (4096, 8192, 2048)])
def test_gemm_swiglu_epilogue(M, H, K):
    """up / gate projections with SwiGLU in the epilogue against fp32 references and, bit for bit, against two plain
    GEMMs followed by the stand-alone SwiGLU kernel (the activation is computed from the rounded up / gate)."""
    from llm_kittens_b200.ops import _native, elementwise as ew, gemm

    torch.manual_seed(M + H)
    a, wu, wg = _rand(M, K), _rand(H, K, scale=0.1), _rand(H, K, scale=0.1)
    act, up, gate = (torch.empty(M, H, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    if not gemm.gemm_swiglu(a, wu, wg, act, up, gate):
        pytest.skip("fused SwiGLU kernel not available for this shape / device")
    _native.check_status()
    ref_up, ref_gate = a.float() @ wu.float().T, a.float() @ wg.float().T
    _close(up, ref_up, 0.02 * max(1.0, ref_up.abs().max().item()))
    _close(gate, ref_gate, 0.02 * max(1.0, ref_gate.abs().max().item()))
    up2, gate2 = gemm.gemm_nt(a, wu), gemm.gemm_nt(a, wg)
    assert torch.equal(up, up2) and torch.equal(gate, gate2)
    assert torch.equal(act, ew.swiglu_fwd(gate2, up2))
