"""Model-FLOPs-utilisation helpers and optional NVML telemetry (``-lg``).

``flops_promised`` returns the dense tensor-core peak for the device name and precision; the
reference's table (llmc/mfu.h:42-102) has no B200 row, this one does (2250 TFLOP/s dense bf16
nominal), and a measured peak file can override it. NVML access is read-only."""
from __future__ import annotations

import json
import os

# dense (no 2:4 sparsity) TFLOP/s by (substring of device name) -> {precision: tflops}
_PEAKS = [
    ("B200", {"bf16": 2250.0, "fp16": 2250.0, "fp8": 4500.0, "tf32": 1100.0}),
    ("GB200", {"bf16": 2500.0, "fp16": 2500.0, "fp8": 5000.0, "tf32": 1250.0}),
    ("H100 PCIe", {"bf16": 756.0, "fp16": 756.0, "tf32": 378.0}),
    ("H100", {"bf16": 989.4, "fp16": 989.4, "tf32": 494.7}),
    ("H200", {"bf16": 989.4, "fp16": 989.4, "tf32": 494.7}),
    ("A100", {"bf16": 312.0, "fp16": 312.0, "tf32": 156.0}),
    ("RTX 5090", {"bf16": 419.0, "fp16": 419.0, "tf32": 209.5}),
    ("RTX 4090", {"bf16": 330.3, "fp16": 330.3, "tf32": 82.6}),
]


def flops_promised(device_name: str, precision: str = "bf16") -> float:
    """Peak TFLOP/s, or -1.0 when the device is unknown."""
    for key, table in _PEAKS:
        if key in device_name:
            return table.get(precision, -1.0)
    return -1.0


def measured_peak_tflops(path: str | None = None) -> float | None:
    """bf16 TFLOP/s from a JSON file with a ``bf16_tflops`` field (a measurement of this machine): ``path`` or the
    file named by ``LLMK_MEASURED_PEAKS``; None when neither is given or the file cannot be read."""
    path = path or os.environ.get("LLMK_MEASURED_PEAKS")
    if not path:
        return None
    try:
        return float(json.load(open(path))["bf16_tflops"])
    except Exception:
        return None


def estimate_flops_per_token(num_parameters: int, num_layers: int, channels: int, seq_len: int,
                             embedding_parameters: int = 0) -> float:
    """6*N + 6*L*C*T (N without the position embedding), the estimate the reference prints as MFU
    (train_gpt2.cu:1381-1408)."""
    n = num_parameters - embedding_parameters
    return 6.0 * n + 6.0 * num_layers * channels * seq_len


def mfu(tokens_per_second: float, flops_per_token: float, peak_tflops: float) -> float:
    if peak_tflops <= 0:
        return -1.0
    return tokens_per_second * flops_per_token / (peak_tflops * 1e12)


def gpu_utilization_info(index: int = 0) -> dict | None:
    """Clock / power / temperature / utilisation / throttle reasons through NVML (read-only)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        util = pynvml.nvmlDeviceGetUtilizationRates(h)
        info = {
            "clock_mhz": pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM),
            "max_clock_mhz": pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM),
            "power_w": pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0,
            "power_limit_w": pynvml.nvmlDeviceGetEnforcedPowerLimit(h) / 1000.0,
            "temperature_c": pynvml.nvmlDeviceGetTemperature(h, pynvml.NVML_TEMPERATURE_GPU),
            "gpu_util": util.gpu,
            "mem_util": util.memory,
            "throttle_reasons": pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h),
        }
        return info
    except Exception:
        return None
