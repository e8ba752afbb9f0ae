"""Parser and thresholds of the kernel-profiling tool (no GPU, no ncu needed)."""
from llm_kittens_b200.cli import profile_kernels as pk

RAW = (
    '"ID","Kernel Name","gpu__time_duration.sum","sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",'
    '"gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed","launch__registers_per_thread"\n'
    '"","","us","%","%","register/thread"\n'
    '"0","void gemm_kernel<0, 1, 1>(...)","170.3","72.4","25.2","145"\n'
)


def test_parse_and_thresholds():
    rows = pk.parse_raw_csv(RAW)
    assert len(rows) == 1 and rows[0]["tensor_pct"] == 72.4 and rows[0]["regs"] == 145
    assert pk.evaluate({"gemm_nt": rows}, 60, 50) == []
    assert pk.evaluate({"gemm_nt": rows}, 80, 50)[0].startswith("gemm_nt: tensor pipe active")
    assert pk.evaluate({"classifier": rows}, 60, 50)[0].startswith("classifier: DRAM")
    assert pk.evaluate({"adamw": []}, 60, 50) == ["adamw: no launch captured"]
