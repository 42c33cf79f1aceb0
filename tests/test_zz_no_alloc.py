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


def _reference_fp32(dy, x, w, rstd, residual):
    """The same backward pass as plain fp32 PyTorch statements."""
    dyf, xf = dy.float(), x.float()
    xhat = xf * rstd[:, None]
    g = dyf * w[None, :]
    dx = rstd[:, None] * (g - xhat * (g * xhat).mean(dim=1, keepdim=True))
    if residual is not None:
        dx = dx + residual.float()
    return dx, (dyf * xhat).sum(dim=0)


CASES = [(1000, 4096, True), (333, 1024, False), (5, 8192, True), (148, 8, False)]


def test_noalloc_matches_regular_entry_point_twice():
    from b200moe.ops import native
    lib = native.require()
    lib.b2_rmsnorm_bwd_noalloc_strerror.restype = ctypes.c_char_p
    torch.manual_seed(11)
    for call, (rows, D, with_residual) in enumerate(CASES):
        x = torch.randn(rows, D, device="cuda").bfloat16()
        dy = torch.randn(rows, D, device="cuda").bfloat16()
        res = torch.randn(rows, D, device="cuda").bfloat16() if with_residual else None
        w = torch.rand(D, device="cuda") + 0.5
        _, rstd = native.rmsnorm_fwd(x, w, 1e-5)
        want_dx, want_dw = native.rmsnorm_bwd(dy, x, w, rstd, residual_grad=res)
        ref_dx, ref_dw = _reference_fp32(dy, x, w, rstd, res)
        dx = torch.empty_like(x)
        dw = torch.empty(D, device="cuda", dtype=torch.float32)
        rc = _call(lib, dy, x, w, rstd, res, dx, dw)      # first call: module load and the symbol look-up
        assert rc == 0, lib.b2_rmsnorm_bwd_noalloc_strerror(rc)
        torch.cuda.synchronize()
        first = (dx.clone(), dw.clone())
        # second call in a row: the device's free memory as the driver reports it (cudaMemGetInfo sees a
        # cudaMalloc made by anybody in the process, which PyTorch's own allocator statistics would not)
        dx.zero_()
        dw.zero_()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call(lib, dy, x, w, rstd, res, dx, dw)
        assert rc == 0, lib.b2_rmsnorm_bwd_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the entry point changed the device's free memory"
        for got_dx, got_dw in (first, (dx, dw)):
            assert _rel(got_dx, want_dx) < 8e-3, f"case {call} vs the regular entry point"
            assert _rel(got_dw, want_dw) < 8e-3, f"case {call} vs the regular entry point"
            assert _rel(got_dx, ref_dx) < 8e-3, f"case {call} vs fp32 PyTorch"
            assert _rel(got_dw, ref_dw) < 8e-3, f"case {call} vs fp32 PyTorch"


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


def test_noalloc_refuses_null_and_misaligned_pointers_before_any_launch():
    from b200moe.ops import native
    lib = native.require()
    lib.b2_rmsnorm_bwd_noalloc_strerror.restype = ctypes.c_char_p
    rows, D = 6, 64
    pool = torch.zeros(rows * D + 8, device="cuda", dtype=torch.bfloat16)
    aligned = pool[:rows * D].view(rows, D)
    shifted = pool[1:rows * D + 1].view(rows, D)          # 2 bytes off the 16-byte grid
    w = torch.ones(D, device="cuda")
    rstd = torch.ones(rows, device="cuda")
    dx = torch.full((rows, D), 7.0, device="cuda", dtype=torch.bfloat16)
    dw = torch.full((D,), 7.0, device="cuda")
    assert shifted.data_ptr() % 16 != 0
    for args in ((shifted, aligned, w, rstd, None, dx, dw), (aligned, shifted, w, rstd, None, dx, dw),
                 (aligned, aligned, w, rstd, shifted, dx, dw)):
        rc = _call(lib, *args)
        assert rc == -8 and b"aligned" in lib.b2_rmsnorm_bwd_noalloc_strerror(rc)
    assert _call(lib, None, aligned, w, rstd, None, dx, dw) == -1
    torch.cuda.synchronize()
    assert float(dx.float().min()) == 7.0 and float(dw.min()) == 7.0      # nothing was written
