"""One small, self-ending workload per kernel for profiler captures:

    python -m llm_kittens_b200.ops.profile_case <case> [launches]

cases: gemm_nt, gemm_nt_gelu, gemm_nn, gemm_tn, attn_fwd, attn_bwd, layernorm_fwd, layernorm_bwd,
classifier, adamw, comm_rs, comm_adamw_push (the peer-memory kernels with all ranks emulated on one GPU).
Each case allocates inputs larger than the L2 (but well under a few GB), runs
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
    if case in ("comm_rs", "comm_adamw_push"):
        # The peer-memory kernels with all P "ranks" emulated on this GPU in ONE launch: P local buffers stand for the
        # peers' buffers and every flag is pre-set, so nothing waits. Shows the kernels' own load / reduce / store
        # rates; the NVLink part cannot be profiled here (multi-rank programs are not run under the profiler).
        import ctypes

        P, L, C = 8, 12, 768
        per_layer = 12 * C * C + 13 * C                       # one GPT-2 block's parameters
        n = L * per_layer
        shard = per_layer // P // 8 * 8
        bufs = [_rnd(n, scale=0.01) for _ in range(P)]
        ptrs = (ctypes.c_longlong * P)(*[int(b.data_ptr()) for b in bufs])
        ctrl = torch.full((int(N.lib().llmk_comm_ctrl_ints()),), 1 << 20, dtype=torch.int32, device="cuda")
        gshard = torch.zeros(L * shard, dtype=torch.float32, device="cuda")
        if case == "comm_rs":
            rows = [(l * per_layer, l * shard, shard) for l in range(L)]       # rank 0's slice of every block
            table = torch.tensor(rows, dtype=torch.int64, device="cuda")
            partials = torch.zeros(len(rows) * 64, dtype=torch.float32, device="cuda")
            return lambda: N.call("llmk_comm_rs_bucket", ptrs, ctrl, 0, 1, table, len(rows), gshard, partials, 64, P, 0,
                                  int(1e9), N.status_word())
        m, v, master = (torch.zeros(L * shard, dtype=torch.float32, device="cuda") for _ in range(3))
        segs = torch.tensor([(l * per_layer, l * shard, shard, 1) for l in range(L)], dtype=torch.int64, device="cuda")
        scale = torch.ones(1, device="cuda")
        return lambda: N.call("llmk_comm_adamw_push", ptrs, master, gshard, m, v, segs, L, shard, 1e-4, 0.9, 0.95, 0.1, 0.05, 1e-8,
                              0.1, scale, 1234, P, 0)
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
