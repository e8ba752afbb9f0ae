"""Profile the hot kernels with Nsight Compute and check their tensor-core / DRAM utilisation.

Same purpose as the reference's profile_gpt2cu.py:14-110 (run ``ncu``, export the raw CSV, average the tensor
pipe activity per kernel class, fail under a threshold), adapted to this code base: every kernel is captured
from a small self-ending case (``ops/profile_case.py``), one launch each, with ``--clock-control none``.

    python -m llm_kittens_b200.cli.profile_kernels --out-dir prof [--cases gemm_nt attn_fwd ...] [--min-tensor 60]

Each case first runs once WITHOUT the profiler and is only captured if that run exits 0.
"""
from __future__ import annotations

import argparse
import csv
import io
import os
import subprocess
import sys

CASES = {  # case -> (kernel regex, class): tensor-core kernels are checked against --min-tensor, the others against --min-dram
    "gemm_nt": ("gemm_kernel", "tensor"),
    "gemm_nt_gelu": ("gemm_kernel", "tensor"),
    "gemm_nn": ("gemm_kernel", "tensor"),
    "gemm_tn": ("gemm_kernel", "tensor"),
    "attn_fwd": ("attn_fwd", "attention"),
    "attn_bwd": ("attn_bwd_dkv", "attention"),
    "layernorm_fwd": ("norm_fwd", "memory"),
    "layernorm_bwd": ("norm_bwd", "memory"),
    "classifier": ("fused_classifier", "memory"),
    "adamw": ("adamw_kernel", "memory"),
}
METRICS = {
    "time_us": "gpu__time_duration.sum",
    "tensor_pct": "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",
    "dram_pct": "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
    "sm_pct": "sm__throughput.avg.pct_of_peak_sustained_elapsed",
    "regs": "launch__registers_per_thread",
}


def parse_raw_csv(text: str) -> list[dict]:
    """Rows of ``ncu --page raw --csv`` -> one dict per captured launch with the METRICS above (floats) and the name."""
    rows = list(csv.reader(io.StringIO(text)))
    if len(rows) < 3:
        return []
    hdr = rows[0]
    out = []
    for r in rows[2:]:
        d = {"kernel": r[hdr.index("Kernel Name")]}
        for key, metric in METRICS.items():
            if metric in hdr:
                try:
                    d[key] = float(r[hdr.index(metric)].replace(",", ""))
                except ValueError:
                    pass
        out.append(d)
    return out


def evaluate(results: dict[str, list[dict]], min_tensor: float, min_dram: float) -> list[str]:
    """Returns the failures (empty = all kernel classes meet their thresholds)."""
    problems = []
    for case, launches in results.items():
        if not launches:
            problems.append(f"{case}: no launch captured")
            continue
        kind = CASES[case][1]
        if kind == "tensor":
            v = sum(l.get("tensor_pct", 0.0) for l in launches) / len(launches)
            if v < min_tensor:
                problems.append(f"{case}: tensor pipe active {v:.1f} % < {min_tensor} %")
        elif kind == "memory":
            v = sum(l.get("dram_pct", 0.0) for l in launches) / len(launches)
            if v < min_dram:
                problems.append(f"{case}: DRAM throughput {v:.1f} % < {min_dram} %")
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out-dir", default="prof")
    ap.add_argument("--cases", nargs="*", default=list(CASES))
    ap.add_argument("--min-tensor", type=float, default=60.0)
    ap.add_argument("--min-dram", type=float, default=50.0)
    args = ap.parse_args(argv)
    os.makedirs(args.out_dir, exist_ok=True)
    results = {}
    for case in args.cases:
        regex, _ = CASES[case]
        base = [sys.executable, "-m", "llm_kittens_b200.ops.profile_case", case, "1"]
        if subprocess.run(base, stdout=subprocess.DEVNULL).returncode != 0:
            print(f"{case}: plain run failed, not profiled")
            results[case] = []
            continue
        rep = os.path.join(args.out_dir, f"{case}.ncu-rep")
        cmd = ["ncu", "--section", "SpeedOfLight", "--section", "LaunchStats", "--clock-control", "none", "-k", f"regex:{regex}",
               "-s", "2", "-c", "1", "-f", "-o", rep[:-8], *base]
        subprocess.run(cmd, stdout=subprocess.DEVNULL, check=False)
        raw = subprocess.run(["ncu", "-i", rep, "--page", "raw", "--csv"], capture_output=True, text=True).stdout
        results[case] = parse_raw_csv(raw)
        for l in results[case]:
            print(f"{case:16s} {l.get('time_us', 0):9.1f} us  tensor {l.get('tensor_pct', 0):5.1f} %  dram {l.get('dram_pct', 0):5.1f} %  "
                  f"sm {l.get('sm_pct', 0):5.1f} %  regs {int(l.get('regs', 0))}  {l['kernel'][:60]}")
    problems = evaluate(results, args.min_tensor, args.min_dram)
    for p in problems:
        print("FAIL", p)
    return 1 if problems else 0


if __name__ == "__main__":
    raise SystemExit(main())
