"""Micro-benchmarks of the attention and the bandwidth-bound kernels (see ``ops/bench.py``)."""
from __future__ import annotations

import torch

from . import _native as N
from .bench import peaks, time_fn

BF = torch.bfloat16


def _rnd(*s, scale=1.0):
    return (torch.randn(*s, device="cuda") * scale).to(BF)


def bench_attention():
    import torch.nn.functional as F

    from . import attention

    tf_peak, _, how = peaks()
    print(f"# causal attention fwd / bwd (ms); FLOPs counted as 4*B*NH*T*T*HS/2 fwd, 2.5x that bwd; peak {tf_peak} TFLOP/s ({how})")
    print(f"{'shape':34s} {'fwd ms':>8s} {'TFLOP/s':>8s} {'bwd ms':>8s} {'TFLOP/s':>8s} {'sdpa fwd':>9s} {'sdpa bwd':>9s}")
    for B, T, NH, NKVH, HS in [(64, 1024, 12, 12, 64), (8, 2048, 32, 8, 64), (1, 4096, 32, 8, 128), (16, 1024, 16, 16, 64)]:
        qkv = _rnd(B, T, (NH + 2 * NKVH) * HS)
        out, lse = attention.attention_fwd(qkv, B, T, NH, NKVH, HS)
        dout = _rnd(B, T, NH * HS)
        dqkv = torch.empty_like(qkv)
        dvec = torch.empty(B, NH, T, dtype=torch.float32, device="cuda")
        tf = time_fn(lambda: attention.attention_fwd(qkv, B, T, NH, NKVH, HS, out=out, lse=lse))
        tfw = time_fn(lambda: attention.attention_fwd(qkv, B, T, NH, NKVH, HS, out=out, lse=lse, impl="warp"))
        tb = time_fn(lambda: attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS, dqkv=dqkv, dvec=dvec))
        tbw = time_fn(lambda: attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NKVH, HS, dqkv=dqkv, dvec=dvec, impl="warp"))
        x = qkv.view(B, T, NH + 2 * NKVH, HS)
        q = x[:, :, :NH].transpose(1, 2).contiguous().requires_grad_(True)
        k = x[:, :, NH:NH + NKVH].transpose(1, 2).contiguous().requires_grad_(True)
        v = x[:, :, NH + NKVH:].transpose(1, 2).contiguous().requires_grad_(True)
        gq = NH != NKVH
        ts = time_fn(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=gq))
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=gq)
        do = torch.randn_like(o)
        tsb = time_fn(lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True))
        fl = 4.0 * B * NH * T * T * HS / 2
        print(f"B{B} T{T} NH{NH} NKVH{NKVH} HS{HS:<14d} {tf:8.3f} (warp {tfw:.3f}) {fl / tf / 1e9:8.1f} {tb:8.3f} (warp {tbw:.3f}) {2.5 * fl / tb / 1e9:8.1f} {ts:9.3f} {tsb:9.3f}")
    N.check_status()


def bench_bandwidth_ops(BT=65536, C=768, V=50257, Vp=50304):
    from . import classifier, elementwise as ew, norm, optim

    _, bw_peak, how = peaks()
    rows = []

    def add(name, nbytes, fn):
        t = time_fn(fn)
        rows.append((name, nbytes, t))

    x, w, b = _rnd(BT, C), _rnd(C) + 1, _rnd(C)
    out = torch.empty_like(x)
    mean, rstd = torch.empty(BT, device="cuda"), torch.empty(BT, device="cuda")
    add("layernorm fwd", 2 * BT * C * 2, lambda: norm.layernorm_fwd(x, w, b, out=out, mean=mean, rstd=rstd))
    res = torch.empty_like(x)
    add("residual+layernorm fwd", 4 * BT * C * 2, lambda: norm.residual_layernorm_fwd(x, out, w, b, residual=res, out=out, mean=mean, rstd=rstd))
    dinp, dw, db = torch.zeros_like(x), torch.zeros(C, device="cuda", dtype=BF), torch.zeros(C, device="cuda", dtype=BF)
    add("layernorm bwd (dinp+=)", 4 * BT * C * 2, lambda: norm.layernorm_bwd(dinp, dw, db, out, x, w, mean, rstd))
    x2, w2 = _rnd(16384, 4096), _rnd(4096) + 1
    o2, r2 = torch.empty_like(x2), torch.empty(16384, device="cuda")
    add("rmsnorm fwd C4096", 2 * x2.numel() * 2, lambda: norm.rmsnorm_fwd(x2, w2, 1e-5, out=o2, rstd=r2))
    d2, dw2 = torch.zeros_like(x2), torch.zeros(4096, device="cuda", dtype=BF)
    add("rmsnorm bwd C4096", 4 * x2.numel() * 2, lambda: norm.rmsnorm_bwd(d2, dw2, o2, x2, w2, r2))
    h = _rnd(BT, 4 * C)
    ho = torch.empty_like(h)
    add("gelu fwd", 2 * h.numel() * 2, lambda: ew.gelu_fwd(h, out=ho))
    add("gelu bwd inplace", 3 * h.numel() * 2, lambda: ew.gelu_bwd_inplace(ho, h))
    add("swiglu fwd", 3 * h.numel() * 2, lambda: ew.swiglu_fwd(h, ho, out=ho))
    dbv = torch.zeros(4 * C, device="cuda", dtype=BF)
    add("dbias OC3072", h.numel() * 2, lambda: ew.dbias(dbv, h))
    dbv2 = torch.zeros(C, device="cuda", dtype=BF)
    add("dbias OC768", x.numel() * 2, lambda: ew.dbias(dbv2, x))
    logits = _rnd(BT, Vp)
    tg = torch.randint(0, V, (BT,), device="cuda", dtype=torch.int32)
    losses = torch.empty(BT, device="cuda")
    add("classifier loss only", logits.numel() * 2, lambda: classifier.fused_classifier(logits, tg, V, 1.0 / BT, losses=losses, write_dlogits=False))
    add("classifier +dlogits", 2 * logits.numel() * 2, lambda: classifier.fused_classifier(logits, tg, V, 1.0 / BT, losses=losses))
    del logits
    n = 124475904
    p, g = _rnd(n, scale=0.02), _rnd(n, scale=0.01)
    m, v, master = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    segs, max_len = optim.make_segments([(0, 0, 0, n, True)])
    scale = torch.ones(1, device="cuda")
    add("adamw (master) 124M", n * (2 + 2 + 2 + 8 + 8 + 8), lambda: optim.adamw(p, master, g, m, v, segs, max_len, 1e-4, 0.9, 0.95, 1, 1e-8, 0.1, scale))
    n2o = torch.zeros(1, device="cuda")
    add("global norm2 124M", n * 2, lambda: optim.global_norm2(g, segs, max_len, out=n2o))
    tok = torch.randint(0, V, (64, 1024), device="cuda", dtype=torch.int32)
    wte, wpe = _rnd(Vp, C), _rnd(1024, C)
    enc = torch.empty(64, 1024, C, device="cuda", dtype=BF)
    add("encoder fwd", 2 * enc.numel() * 2, lambda: ew.encoder_fwd(tok, wte, wpe, out=enc))
    dwte, dwpe = torch.zeros_like(wte), torch.zeros_like(wpe)
    add("encoder bwd (incl. sort)", enc.numel() * 2 * 2, lambda: ew.encoder_bwd(dwte, dwpe, enc, tok))
    print(f"# bandwidth-bound kernels; peak {bw_peak} GB/s ({how}); bytes = algorithmic minimum")
    print(f"{'kernel':34s} {'MB':>9s} {'ms':>8s} {'GB/s':>8s} {'frac':>6s}")
    for name, nb, t in rows:
        gbs = nb / (t * 1e-3) / 1e9
        print(f"{name:34s} {nb / 1e6:9.1f} {t:8.3f} {gbs:8.0f} {gbs / bw_peak:6.2f}")
    N.check_status()
