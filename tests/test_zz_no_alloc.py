"""The allocation-free RMSNorm backward entry point, called through its exported
C symbol, against the regular entry point.

Some callers of the library cannot allocate device memory (code being captured
into a CUDA graph, stream callbacks, hosts with their own memory pool), so
``b2_rmsnorm_bwd_noalloc`` keeps its scratch in a fixed array inside the library.
This file is named to be collected last, so a failure here cannot hide another
test's result in a run that stops at the first failure.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, dy, x, w, rstd, residual, dx, dw):
    fn = lib.b2_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    ptr = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())  # noqa: E731
    return fn(ptr(dy), ptr(x), ptr(w), ptr(rstd), ptr(residual), ptr(dx), ptr(dw), ctypes.c_int(x.shape[0]),
              ctypes.c_int(x.shape[1]), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def test_noalloc_matches_regular_entry_point_twice():
    from b200moe.ops import native
    lib = native.require()
    lib.b2_rmsnorm_bwd_noalloc_strerror.restype = ctypes.c_char_p
    torch.manual_seed(11)
    for call, (rows, D, with_residual) in enumerate([(1000, 4096, True), (333, 1024, False)]):
        x = torch.randn(rows, D, device="cuda").bfloat16()
        dy = torch.randn(rows, D, device="cuda").bfloat16()
        res = torch.randn(rows, D, device="cuda").bfloat16() if with_residual else None
        w = torch.rand(D, device="cuda") + 0.5
        _, rstd = native.rmsnorm_fwd(x, w, 1e-5)
        want_dx, want_dw = native.rmsnorm_bwd(dy, x, w, rstd, residual_grad=res)
        dx = torch.empty_like(x)
        dw = torch.empty(D, device="cuda", dtype=torch.float32)
        before = torch.cuda.memory_allocated()
        rc = _call(lib, dy, x, w, rstd, res, dx, dw)
        assert rc == 0, lib.b2_rmsnorm_bwd_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert _rel(dx, want_dx) < 8e-3, f"call {call}"
        assert _rel(dw, want_dw) < 8e-3, f"call {call}"


def test_noalloc_refuses_sizes_beyond_its_scratch():
    from b200moe.ops import native
    lib = native.require()
    lib.b2_rmsnorm_bwd_noalloc_strerror.restype = ctypes.c_char_p
    rows, D = 4, 8192 + 8
    x = torch.zeros(rows, D, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(D, device="cuda")
    rstd = torch.ones(rows, device="cuda")
    dx = torch.full_like(x, 7.0)
    dw = torch.zeros(D, device="cuda")
    rc = _call(lib, x, x, w, rstd, None, dx, dw)
    assert rc == -3 and b"exceeds" in lib.b2_rmsnorm_bwd_noalloc_strerror(rc)
    torch.cuda.synchronize()
    assert float(dx.float().min()) == 7.0          # nothing was launched
    assert _call(lib, x[:, :12], x[:, :12], w, rstd, None, dx, dw) == -2
