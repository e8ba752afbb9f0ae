"""Optimizer kernels driven by a segment table (``csrc/optim.cu``). Reference jobs: adamw_update,
init_from_master (llmc/adamw.cuh:113-171), global_norm_squared (llmc/global_norm.cuh:77-101)."""
from __future__ import annotations

import torch

from . import _native as N

SEG_FIELDS = 5


def make_segments(rows, device="cuda") -> tuple[torch.Tensor, int]:
    """``rows``: iterable of (param_off, grad_off, state_off, length, weight_decay?) -> (int64 table, max length)."""
    rows = [(int(p), int(g), int(s), int(n), int(bool(wd))) for p, g, s, n, wd in rows if n > 0]
    if any(x % 4 for r in rows for x in r[:4]):
        raise ValueError("segment offsets and lengths must be multiples of 4 elements")
    t = torch.tensor(rows, dtype=torch.int64).reshape(-1, SEG_FIELDS)
    return t.to(device), max(r[3] for r in rows)


def global_norm2(grads, segs, max_len, out=None, partials=None):
    nseg = segs.shape[0]
    gx = int(N.lib().llmk_optim_grid_x(max_len))
    out = torch.empty(1, dtype=torch.float32, device=grads.device) if out is None else out
    if partials is None or partials.numel() < gx * nseg:
        partials = torch.empty(gx * nseg, dtype=torch.float32, device=grads.device)
    N.call("llmk_global_norm2", out, partials, grads, int(grads.dtype == torch.float32), segs, nseg, max_len)
    return out


def clip_scale(norm2, clip, scale_out, norm_out, flag_out=None):
    N.call("llmk_clip_scale", scale_out, norm_out, flag_out, norm2, float(clip))


def adamw(params, master, grads, m, v, segs, max_len, lr, beta1, beta2, step, eps, wd, grad_scale_ptr=None,
          grad_scale=1.0, seed=0):
    b1c = 1.0 - beta1 ** step
    b2c = 1.0 - beta2 ** step
    N.call("llmk_adamw", params, master, grads, int(grads.dtype == torch.float32), m, v, segs, segs.shape[0], max_len,
           float(lr), float(beta1), float(beta2), float(b1c), float(b2c), float(eps), float(wd), grad_scale_ptr,
           float(grad_scale), int(seed) & 0xFFFFFFFF)


def master_from_params(master, params, segs, max_len):
    N.call("llmk_master_from_params", master, params, segs, segs.shape[0], max_len)


def params_from_master(params, master, segs, max_len, seed):
    N.call("llmk_params_from_master", params, master, segs, segs.shape[0], max_len, int(seed) & 0xFFFFFFFF)
