"""Per-kernel micro-benchmarks: ``python -m llm_kittens_b200.ops.bench [gemm|attention|norm|classifier|optim|all]``.

Timing follows the same rules as the end-to-end bench: warm-up iterations, CUDA events on the
launching stream, an L2 flush (a 256 MiB write) between timed iterations, median of the samples.
Each row prints the achieved TFLOP/s or GB/s and its fraction of the measured peaks in the JSON file named by
``LLMK_MEASURED_PEAKS`` (fields ``bf16_tflops``, ``hbm_gbs``; a file of that name in the current directory is
also picked up), else of 1590 TFLOP/s / 6650 GB/s.
The cuBLAS / SDPA columns are the library baselines the hand-written kernels are compared to.
"""
from __future__ import annotations

import json
import os
import statistics
import sys

import torch

from . import _native as N


def peaks():
    p = os.environ.get("LLMK_MEASURED_PEAKS", "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    N.call("llmk_flush_l2", _FLUSH, _FLUSH.numel())


def time_fn(fn, warmup=3, iters=10):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(iters):
        flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        samples.append(s.elapsed_time(e))
    return statistics.median(samples)


def bench_gemm(BT=65536):
    from . import gemm

    tf_peak, _, how = peaks()
    C, V = 768, 50304
    rows = []

    def rnd(*s):
        return (torch.randn(*s, device="cuda") * 0.05).to(torch.bfloat16)

    shapes_nt = [("qkv", BT, 3 * C, C), ("attproj", BT, C, C), ("fc+gelu", BT, 4 * C, C), ("fcproj", BT, C, 4 * C),
                 ("lmhead", BT, V, C), ("llama8b qkv", 8192, 6144, 4096), ("llama8b up", 8192, 14336, 4096),
                 ("llama8b down", 8192, 4096, 14336)]
    for name, M, Nn, K in shapes_nt:
        a, b, bias = rnd(M, K), rnd(Nn, K), rnd(Nn)
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device="cuda")
        pre = torch.empty_like(out) if "gelu" in name else None
        t = time_fn(lambda: gemm.gemm_nt(a, b, bias=bias, out=out, gelu_pre_out=pre))
        t_ref = time_fn(lambda: torch.addmm(bias, a, b.T, out=out))
        rows.append(("NT " + name, M, Nn, K, t, t_ref))
        del a, b, out, pre
    shapes_nn = [("d qkv", BT, C, 3 * C), ("d fc (dgelu src)", BT, C, 4 * C), ("d fcproj+dgelu", BT, 4 * C, C), ("d lmhead", BT, C, V)]
    for name, M, Nn, K in shapes_nn:
        a, b = rnd(M, K), rnd(K, Nn)
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device="cuda")
        aux = rnd(M, Nn) if "dgelu" in name and "src" not in name else None
        t = time_fn(lambda: gemm.gemm_nn(a, b, out=out, dgelu_of=aux))
        t_ref = time_fn(lambda: torch.matmul(a, b, out=out))
        rows.append(("NN " + name, M, Nn, K, t, t_ref))
        del a, b, out
    shapes_tn = [("dW qkv", 3 * C, C, BT), ("dW attproj", C, C, BT), ("dW fc", 4 * C, C, BT), ("dW fcproj", C, 4 * C, BT),
                 ("dW lmhead", V, C, BT)]
    for name, M, Nn, K in shapes_tn:
        a, b = rnd(K, M), rnd(K, Nn)
        out = torch.zeros(M, Nn, dtype=torch.bfloat16, device="cuda")
        t = time_fn(lambda: gemm.gemm_tn(a, b, out=out, accumulate=True))
        t_ref = time_fn(lambda: torch.matmul(a.T, b, out=out))
        rows.append(("TN " + name, M, Nn, K, t, t_ref))
        if name != "dW lmhead" and gemm.fused_dbias_available():
            # the same product with the bias gradient from the same launch, beside dW + the stand-alone column sums
            from . import elementwise as ew

            db = torch.zeros(M, dtype=torch.bfloat16, device="cuda")
            t_f = time_fn(lambda: gemm.gemm_tn(a, b, out=out, accumulate=True, dbias=db))
            t_s = time_fn(lambda: ew.dbias(db, a, accumulate=True))
            rows.append(("TN " + name + " +dbias", M, Nn, K, t_f, t + t_s))
        del a, b, out
    if gemm.fused_drow_available(64):
        # dO = dres W with the attention backward's D = rowsum(dO * O) in the epilogue, beside the GEMM + the pre-pass
        from . import attention

        B_, T_, NH_ = BT // 1024, 1024, C // 64
        a, b, o = rnd(BT, C), rnd(C, C), rnd(BT, C)
        out = torch.empty(BT, C, dtype=torch.bfloat16, device="cuda")
        dvec = torch.empty(B_, NH_, T_, dtype=torch.float32, device="cuda")
        t_f = time_fn(lambda: gemm.gemm_nn(a, b, out=out, drow_of=(o, dvec, T_)))
        t_g = time_fn(lambda: gemm.gemm_nn(a, b, out=out))
        t_p = time_fn(lambda: attention.attention_bwd_prep(out, o, dvec, B_, T_, NH_, 64))
        rows.append(("NN d attproj +D", BT, C, C, t_f, t_g + t_p))
        del a, b, o, out
    N.check_status()
    print(f"# GEMM (tcgen05) vs cuBLAS; peak {tf_peak} TFLOP/s bf16 ({how}); for the '+dbias' and '+D' rows the last two")
    print("# columns compare with this library's own unfused pair of kernels instead of cuBLAS")
    print(f"{'shape':28s} {'M':>6s} {'N':>6s} {'K':>6s} {'ms':>8s} {'TFLOP/s':>8s} {'frac':>6s} {'cublas ms':>9s} {'ratio':>6s}")
    for name, M, Nn, K, t, t_ref in rows:
        tf = 2.0 * M * Nn * K / (t * 1e-3) / 1e12
        print(f"{name:28s} {M:6d} {Nn:6d} {K:6d} {t:8.3f} {tf:8.1f} {tf / tf_peak:6.2f} {t_ref:9.3f} {t_ref / t:6.2f}")


def step_ledger(model_desc="d12", B=64, T=1024, total_batch=524288):
    """Where one optimizer step of the headline configuration spends its device time: the step runs eagerly with
    every library call between two CUDA events (no profiler), so each kernel is timed inside the step, at the
    clocks the step really runs at. Printed beside the same step without events and replayed from a CUDA graph."""
    import subprocess
    import threading
    import time

    from ..models.config import config_from_descriptor
    from ..models.transformer import Transformer
    from ..runtime.trainer import Trainer

    cfg = config_from_descriptor(model_desc)
    model = Transformer(cfg, device=torch.device("cuda"), recompute=0)
    model.init_weights(42)
    tr = Trainer(model, learning_rate=6e-4, weight_decay=0.1)
    accum = total_batch // (B * T)
    g = torch.Generator().manual_seed(1337)
    batches = [(torch.randint(0, cfg.vocab_size, (B, T), generator=g, dtype=torch.int32).cuda(),
                torch.randint(0, cfg.vocab_size, (B, T), generator=g, dtype=torch.int32).cuda()) for _ in range(accum)]
    clocks = []
    smi = subprocess.Popen(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits", "-lms", "200",
                            "-i", str(torch.cuda.current_device())], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
    threading.Thread(target=lambda: [clocks.append((time.time(), ln)) for ln in smi.stdout], daemon=True).start()

    def step():
        tr.accumulate(batches)
        tr.update(6e-4)

    def timed(n):
        torch.cuda.synchronize()
        w0 = time.time()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            step()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / n, w0, time.time()

    def median_clock(w0, w1):
        v = [float(ln.split(",")[0]) for ts, ln in clocks if w0 <= ts <= w1 and ln.strip()]
        return statistics.median(v) if v else float("nan")

    for _ in range(3):
        step()
    eager_ms, w0, w1 = timed(3)
    eager_clk = median_clock(w0, w1)
    N.ledger_start()
    led_ms, w0, w1 = timed(2)
    rows = N.ledger_stop()
    led_clk = median_clock(w0, w1)
    tr.enable_cuda_graph(True)
    for _ in range(2):
        step()
    graph_ms, w0, w1 = timed(3)
    graph_clk = median_clock(w0, w1)
    smi.terminate()
    N.check_status()
    print(f"# step ledger: {model_desc} B={B} T={T} total batch {total_batch} ({accum} micro-steps), 1 GPU")
    print(f"step, eager launches: {eager_ms:8.2f} ms   (median SM clock {eager_clk:.0f} MHz)")
    print(f"step, eager + events: {led_ms:8.2f} ms   (median SM clock {led_clk:.0f} MHz)")
    print(f"step, CUDA graph    : {graph_ms:8.2f} ms   (median SM clock {graph_clk:.0f} MHz)")
    total = sum(ms for _, ms in rows.values()) / 2
    print(f"{'entry point / GEMM shape':52s} {'calls/step':>10s} {'ms/step':>9s} {'share':>6s} {'us/call':>8s}")
    for label, (n, ms) in sorted(rows.items(), key=lambda kv: -kv[1][1]):
        print(f"{label:52s} {n // 2:10d} {ms / 2:9.3f} {ms / 2 / total:6.1%} {1e3 * ms / n:8.1f}")
    print(f"{'sum of the bracketed calls':52s} {'':10s} {total:9.3f}")
    print(f"{'outside the brackets (gaps, torch ops, events)':52s} {'':10s} {led_ms - total:9.3f}")


def main(argv):
    what = argv[1] if len(argv) > 1 else "all"
    if what == "ledger":
        step_ledger()
        return
    if what in ("gemm", "all"):
        bench_gemm()
    if what in ("attention", "all"):
        from .bench_more import bench_attention
        bench_attention()
    if what in ("elementwise", "norm", "classifier", "optim", "all"):
        from .bench_more import bench_bandwidth_ops
        bench_bandwidth_ops()


if __name__ == "__main__":
    main(sys.argv)
