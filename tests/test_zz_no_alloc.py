"""The allocation-free LayerNorm backward (``llmk_layernorm_bwd_noalloc``), called through its exported
C symbol, must give what the ordinary entry point gives. It serves callers that may not allocate device
memory (no cudaMalloc, no PyTorch allocator) while they drive the kernels: its temporary buffer is a
fixed array inside the library that every call shares, so the test runs two calls back to back with
different shapes and checks that the second is not disturbed by what the first left behind, and that a
shape too large for the built-in buffer is refused with an error code instead of being launched.

This file is collected last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
LLMK_ERR_LIMIT = -6


def _call_noalloc(lib, dinp, dw, db, dout, x, w, mean, rstd, accumulate):
    fn = lib.llmk_layernorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    N, C = x.shape
    return fn(dinp.data_ptr(), dw.data_ptr(), db.data_ptr(), dout.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(),
              rstd.data_ptr(), N, C, int(accumulate), torch.cuda.current_stream().cuda_stream)


def _case(N, C, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(N, C, device="cuda", generator=g).to(BF)
    w = (torch.randn(C, device="cuda", generator=g) * 0.5 + 1).to(BF)
    dout = torch.randn(N, C, device="cuda", generator=g).to(BF)
    mean = x.float().mean(-1)
    rstd = torch.rsqrt(x.float().var(-1, unbiased=False) + 1e-5)
    dinp0 = torch.randn(N, C, device="cuda", generator=g).to(BF)
    return x, w, dout, mean, rstd, dinp0


def test_noalloc_layernorm_backward_matches_allocating_entry_point_twice():
    from llm_kittens_b200.ops import _native, norm

    lib = _native.lib()
    for N, C, seed in ((1000, 768, 1), (333, 1024, 2)):   # two calls in a row, second with another shape
        x, w, dout, mean, rstd, dinp0 = _case(N, C, seed)
        ref_dinp, ref_dw, ref_db = dinp0.clone(), torch.zeros(C, device="cuda", dtype=BF), torch.zeros(C, device="cuda", dtype=BF)
        norm.layernorm_bwd(ref_dinp, ref_dw, ref_db, dout, x, w, mean, rstd, accumulate_dinp=True)
        got_dinp, got_dw, got_db = dinp0.clone(), torch.zeros(C, device="cuda", dtype=BF), torch.zeros(C, device="cuda", dtype=BF)
        rc = _call_noalloc(lib, got_dinp, got_dw, got_db, dout, x, w, mean, rstd, True)
        assert rc == 0
        torch.cuda.synchronize()
        assert (got_dinp.float() - ref_dinp.float()).abs().max().item() <= 0.06
        assert (got_dw.float() - ref_dw.float()).abs().max().item() <= 0.02 * max(1.0, ref_dw.float().abs().max().item())
        assert (got_db.float() - ref_db.float()).abs().max().item() <= 0.02 * max(1.0, ref_db.float().abs().max().item())
        # against the PyTorch fp32 formula as well
        xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
        bf = torch.zeros(C, device="cuda", requires_grad=True)
        torch.nn.functional.layer_norm(xf, (C,), wf, bf, 1e-5).backward(dout.float())
        assert (got_dinp.float() - (xf.grad + dinp0.float())).abs().max().item() < 0.08
        assert (got_dw.float() - wf.grad).abs().max().item() < 0.02 * max(1.0, wf.grad.abs().max().item())


def test_noalloc_rejects_shapes_beyond_the_builtin_buffer():
    from llm_kittens_b200.ops import _native

    lib = _native.lib()
    N, C = 8, 6144   # needs 4 * SMs * 2 * C floats, more than the 4 Mi floats inside the library
    x, w, dout, mean, rstd, dinp0 = _case(N, C, 3)
    dw, db = torch.zeros(C, device="cuda", dtype=BF), torch.zeros(C, device="cuda", dtype=BF)
    before = dinp0.clone()
    assert _call_noalloc(lib, dinp0, dw, db, dout, x, w, mean, rstd, True) == LLMK_ERR_LIMIT
    torch.cuda.synchronize()
    assert torch.equal(dinp0, before) and dw.abs().max().item() == 0
