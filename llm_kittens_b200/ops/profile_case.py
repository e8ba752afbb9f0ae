"""One small, self-ending workload per kernel for profiler captures:

    python -m llm_kittens_b200.ops.profile_case <case> [launches]

cases: gemm_nt, gemm_nt_gelu, gemm_nn, gemm_tn, attn_fwd, attn_bwd, layernorm_fwd, layernorm_bwd,
classifier, adamw. Each case allocates inputs larger than the L2 (but well under a few GB), runs
the op twice as warm-up and then `launches` (default 2) more times, and checks the status word.
Used as ``ncu --set full --clock-control none -k regex:<kernel> -s <warm-up launches> -c 1 ...``.
"""
from __future__ import annotations

import sys

import torch

from . import _native as N

BF = torch.bfloat16


def _rnd(*s, scale=1.0):
    return (torch.randn(*s, device="cuda") * scale).to(BF)


def build(case: str):
    from . import attention, classifier, gemm, norm, optim

    BT, C = 65536, 768
    if case == "gemm_nt":
        a, b, bias, out = _rnd(BT, C), _rnd(3 * C, C, scale=0.05), _rnd(3 * C), torch.empty(BT, 3 * C, device="cuda", dtype=BF)
        return lambda: gemm.gemm_nt(a, b, bias=bias, out=out)
    if case == "gemm_nt_gelu":
        a, b, bias = _rnd(BT, C), _rnd(4 * C, C, scale=0.05), _rnd(4 * C)
        out, pre = torch.empty(BT, 4 * C, device="cuda", dtype=BF), torch.empty(BT, 4 * C, device="cuda", dtype=BF)
        return lambda: gemm.gemm_nt(a, b, bias=bias, out=out, gelu_pre_out=pre)
    if case == "gemm_nn":
        a, b, out = _rnd(BT, 3 * C), _rnd(3 * C, C, scale=0.05), torch.empty(BT, C, device="cuda", dtype=BF)
        return lambda: gemm.gemm_nn(a, b, out=out)
    if case == "gemm_tn":
        a, b, out = _rnd(BT, 4 * C, scale=0.1), _rnd(BT, C, scale=0.1), torch.zeros(4 * C, C, device="cuda", dtype=BF)
        return lambda: gemm.gemm_tn(a, b, out=out, accumulate=True)
    if case in ("attn_fwd", "attn_bwd"):
        B, T, NH, HS = 64, 1024, 12, 64
        qkv = _rnd(B, T, 3 * NH * HS)
        out, lse = attention.attention_fwd(qkv, B, T, NH, NH, HS)
        dout, dqkv = _rnd(B, T, NH * HS), torch.empty_like(qkv)
        dvec = torch.empty(B, NH, T, dtype=torch.float32, device="cuda")
        if case == "attn_fwd":
            return lambda: attention.attention_fwd(qkv, B, T, NH, NH, HS, out=out, lse=lse)
        return lambda: attention.attention_bwd(dout, qkv, out, lse, B, T, NH, NH, HS, dqkv=dqkv, dvec=dvec)
    if case in ("layernorm_fwd", "layernorm_bwd"):
        x, w, b = _rnd(BT * 2, C), _rnd(C) + 1, _rnd(C)
        out = torch.empty_like(x)
        mean, rstd = torch.empty(BT * 2, device="cuda"), torch.empty(BT * 2, device="cuda")
        norm.layernorm_fwd(x, w, b, out=out, mean=mean, rstd=rstd)
        if case == "layernorm_fwd":
            return lambda: norm.layernorm_fwd(x, w, b, out=out, mean=mean, rstd=rstd)
        dinp, dw, db = torch.zeros_like(x), torch.zeros(C, device="cuda", dtype=BF), torch.zeros(C, device="cuda", dtype=BF)
        return lambda: norm.layernorm_bwd(dinp, dw, db, out, x, w, mean, rstd)
    if case == "classifier":
        rows, V, Vp = 8192, 50257, 50304
        logits = _rnd(rows, Vp)
        tg = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
        losses = torch.empty(rows, device="cuda")
        return lambda: classifier.fused_classifier(logits, tg, V, 1.0 / rows, losses=losses)
    if case == "adamw":
        n = 124475904
        p, g = _rnd(n, scale=0.02), _rnd(n, scale=0.01)
        m, v, master = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
        segs, max_len = optim.make_segments([(0, 0, 0, n, True)])
        scale = torch.ones(1, device="cuda")
        return lambda: optim.adamw(p, master, g, m, v, segs, max_len, 1e-4, 0.9, 0.95, 1, 1e-8, 0.1, scale)
    raise SystemExit(f"unknown case {case}")


def main(argv):
    case = argv[1]
    launches = int(argv[2]) if len(argv) > 2 else 2
    fn = build(case)
    for _ in range(2 + launches):
        fn()
    torch.cuda.synchronize()
    N.check_status()
    print(f"{case}: ok")


if __name__ == "__main__":
    main(sys.argv)
