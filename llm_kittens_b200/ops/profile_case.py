"""One small, self-ending workload per kernel for profiler captures:

    python -m llm_kittens_b200.ops.profile_case <case> [launches]

cases: gemm_nt, gemm_nt_gelu, gemm_nn, gemm_tn, gemm_tn_dbias (weight and bias gradient from one launch), gemm_nn_drow (dO and the attention backward's row sums), attn_fwd, attn_bwd, layernorm_fwd, layernorm_bwd,
classifier, adamw, comm_rs, comm_adamw_push, comm_ag_flags (the peer-memory kernels with all ranks emulated on one GPU),
gemm_b_ready (the GEMM that polls the flags of a gathered weight, flags already set), gemm_qkv_rope (QKV projection with
RoPE in the epilogue), moe_dispatch / moe_grouped_a_ready / moe_dispatch_pull / moe_combine_pull (the expert exchange with
its arrival table, ranks emulated).
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
    if case == "gemm_nn_drow":
        B, T, NH = 64, 1024, 12
        a, b, o = _rnd(BT, C), _rnd(C, C, scale=0.05), _rnd(BT, C)
        out, dvec = torch.empty(BT, C, device="cuda", dtype=BF), torch.empty(B, NH, T, device="cuda")
        return lambda: gemm.gemm_nn(a, b, out=out, drow_of=(o, dvec, T))
    if case == "gemm_tn_dbias":
        a, b, out = _rnd(BT, 4 * C, scale=0.1), _rnd(BT, C, scale=0.1), torch.zeros(4 * C, C, device="cuda", dtype=BF)
        db = torch.zeros(4 * C, device="cuda", dtype=BF)
        return lambda: gemm.gemm_tn(a, b, out=out, accumulate=True, dbias=db)
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
    if case == "comm_ag_flags":
        # the tile-granular gather of one Llama-3 8B block's matrices from 8 "ranks" that are 8 local buffers
        import ctypes

        P = 8
        tensors = [4096 * 6144, 4096 * 4096, 4096 * 14336, 4096 * 14336, 14336 * 4096]
        shard_total = sum(t // P for t in tensors)
        shards = [_rnd(shard_total, scale=0.02) for _ in range(P)]
        ptrs = (ctypes.c_longlong * P)(*[int(b.data_ptr()) for b in shards])
        staging = torch.empty(sum(tensors), dtype=BF, device="cuda")
        rows, off, s_off, nflags = [], 0, 0, 0
        for size in tensors:
            ln = size // P
            cps = max(1, min(8, ln // (1 << 19)))
            while cps > 1 and ln % (cps * 8):
                cps -= 1
            rows.append((s_off, off, ln, nflags, cps))
            nflags += P * cps
            off += size
            s_off += ln
        table = torch.tensor(rows, dtype=torch.int64, device="cuda")
        flags, arrivals = torch.zeros(nflags, dtype=torch.int32, device="cuda"), torch.zeros(nflags, dtype=torch.int32, device="cuda")
        tick = [0]

        def run():
            tick[0] += 1
            N.call("llmk_comm_ag_bucket_flags", ptrs, staging, table, len(rows), max(r[4] for r in rows), P, flags, arrivals,
                   max(1, min(16, 600 // nflags)), tick[0])

        return run
    if case == "gemm_b_ready":
        M, Nn, K = 8192, 6144, 4096                      # Llama-3 8B QKV projection on 8192 tokens
        a, w, out = _rnd(M, K), _rnd(Nn, K, scale=0.02), torch.empty(M, Nn, device="cuda", dtype=BF)
        chunk = 524288
        flags = torch.full(((Nn * K) // chunk,), 5, dtype=torch.int32, device="cuda")
        entry = gemm.register_b_ready(w, flags, 0, chunk, int(1e9))
        entry[3] = 5
        return lambda: gemm.gemm_nt(a, w, out=out)
    if case == "gemm_qkv_rope":
        from . import elementwise as ew

        B, T, NH, NKVH, HS, Cc = 2, 4096, 32, 8, 128, 4096
        x, w = _rnd(B * T, Cc), _rnd((NH + 2 * NKVH) * HS, Cc, scale=0.02)
        out = torch.empty(B * T, (NH + 2 * NKVH) * HS, device="cuda", dtype=BF)
        table = ew.rope_tables(T, HS, 500000.0, False)
        return lambda: gemm.gemm_qkv_rope(x, w, table, T, (NH + NKVH) * HS, HS, out=out)
    if case in ("moe_dispatch_pull", "moe_combine_pull"):
        # the pull-style expert exchange at the d24 shape with this GPU as every rank: the owner-side dispatch that fetches
        # routed rows through the inverse slot map, and the combine that fetches expert outputs; flags pre-set
        from . import moe as moe_ops

        Ntok, Cc, E, K = 16384, 1024, 8, 2
        cap = (int(-(-1.25 * K * Ntok // E)) + 7) // 8 * 8
        x, wr = _rnd(Ntok, Cc), _rnd(E, Cc, scale=0.5)
        probs, idx, tw = moe_ops.router_fwd(x, wr, K)
        slot, counts = moe_ops.assign_slots(idx, E, cap)
        inv_tok = torch.empty(E * cap, dtype=torch.int32, device="cuda")
        inv_w = torch.empty(E * cap, dtype=torch.float32, device="cuda")
        moe_ops.inverse_map(inv_tok, inv_w, idx, slot, tw, E, cap)
        recv = torch.zeros(E * cap, Cc, dtype=BF, device="cuda")
        ready = torch.full((2 * E,), 1 << 20, dtype=torch.int32, device="cuda")
        done = torch.zeros(E, dtype=torch.int32, device="cuda")
        out = torch.empty(Ntok, Cc, dtype=BF, device="cuda")
        save = torch.empty(E * cap, Cc, dtype=BF, device="cuda")
        tab = lambda t: moe_ops.ptr_table([t])
        if case == "moe_dispatch_pull":
            return lambda: moe_ops.dispatch_pull(recv, tab(x), tab(inv_tok), tab(inv_w), Cc, E, cap, 0, 1, False, ready, done, 1, int(1e9))
        return lambda: moe_ops.combine_pull(out, x, tab(recv), save, idx, slot, tw, E, cap, 0, 1, ready, 1, int(1e9))
    if case in ("moe_dispatch", "moe_grouped_a_ready"):
        # one MoE layer's exchange at the d24 shape (C=1024, H=4096, 8 experts, top-2, 16384 tokens): this GPU plays all
        # ranks (a one-entry peer table), so dispatch, arrival table and the waiting GEMM are exercised without a peer
        from . import moe as moe_ops

        Ntok, Cc, H, E, K = 16384, 1024, 4096, 8, 2
        cap = int(-(-1.25 * K * Ntok // E))
        cap = (cap + 7) // 8 * 8
        x, wr = _rnd(Ntok, Cc), _rnd(E, Cc, scale=0.5)
        probs, idx, tw = moe_ops.router_fwd(x, wr, K)
        slot, counts = moe_ops.assign_slots(idx, E, cap)
        recv = torch.zeros(E * cap, Cc, dtype=BF, device="cuda")
        arrive = torch.zeros(E, dtype=torch.int32, device="cuda")
        done = torch.zeros(1, dtype=torch.int32, device="cuda")
        ep = [0]
        w1, b1 = _rnd(E * H, Cc, scale=0.02), _rnd(E * H)
        act, pre = torch.empty(E * cap, H, dtype=BF, device="cuda"), torch.empty(E * cap, H, dtype=BF, device="cuda")

        def run():
            ep[0] += 1
            moe_ops.dispatch_signal(moe_ops.ptr_table([recv]), x, idx, slot, tw, counts, E, cap, 0, 1, False, moe_ops.ptr_table([arrive]),
                                    0, done, ep[0])
            if case == "moe_grouped_a_ready":
                gemm.gemm_nt(recv, w1, bias=b1, out=act, gelu_pre_out=pre, groups=E, a_ready=(arrive, cap, ep[0], int(1e9)))

        return run
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
