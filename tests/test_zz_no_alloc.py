"""The allocation-free RMSNorm backward entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory at the time of the call (fixed memory budgets,
plug-ins working on a host application's stream, loops that must never hit cudaMalloc).  For them the library
exports ``jpb_rmsnorm_bwd_noalloc``, which keeps its scratch in a fixed array inside the library.  This file
checks it against the regular entry point (``jpb_norm_bwd`` with a caller-provided scratch tensor) on two
calls in a row, and checks that oversized rows are refused.  It is named to be collected last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from jaxpp_b200.ops import native

    lib = native.load()
    p, i = ctypes.c_void_p, ctypes.c_int
    lib.jpb_rmsnorm_bwd_noalloc.argtypes = [i, p, p, p, p, p, p, i, i, p]
    lib.jpb_rmsnorm_bwd_noalloc.restype = i
    lib.jpb_noalloc_strerror.argtypes = [i]
    lib.jpb_noalloc_strerror.restype = ctypes.c_char_p
    return lib, native


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_matches_regular_entry_point_twice(dtype):
    lib, native = _lib()
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    stream = torch.cuda.current_stream().cuda_stream
    # the second call reuses the array with another shape; the third repeats the second: by then every kernel it
    # launches has been loaded, so the driver's own count of free device memory must not move either
    for call, (rows, H) in enumerate([(300, 4096), (37, 1024), (37, 1024)]):
        g = torch.Generator(device="cuda").manual_seed(100 + call)
        x = torch.randn(rows, H, generator=g, device="cuda").to(dtype)
        dy = torch.randn(rows, H, generator=g, device="cuda").to(dtype)
        w = torch.randn(H, generator=g, device="cuda").to(dtype)
        _, rstd = native.rmsnorm(x, w, 1e-5)
        ref_dx, ref_dw = native.rmsnorm_bwd(dy, x, w, rstd)
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        before = torch.cuda.memory_allocated()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.jpb_rmsnorm_bwd_noalloc(0 if dtype == torch.float32 else 1, dy.data_ptr(), x.data_ptr(), w.data_ptr(),
                                         rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, H, stream)
        assert rc == 0, lib.jpb_noalloc_strerror(rc).decode()
        assert torch.cuda.memory_allocated() == before  # nothing went through torch's allocator ...
        torch.cuda.synchronize()
        if call == 2:                                   # ... and nothing past it (a raw cudaMalloc would show here)
            assert torch.cuda.mem_get_info()[0] >= free_before
        torch.testing.assert_close(dx.float(), ref_dx.float(), **tol)
        torch.testing.assert_close(dw.float(), ref_dw.float(), rtol=tol["rtol"], atol=tol["atol"] * rows ** 0.5)


def test_noalloc_rejects_rows_longer_than_the_builtin_scratch():
    lib, _ = _lib()
    t = torch.zeros(8, device="cuda")
    rc = lib.jpb_rmsnorm_bwd_noalloc(0, t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                     4, 16384, None)
    assert rc == -20 and b"8192" in lib.jpb_noalloc_strerror(rc)
    rc = lib.jpb_rmsnorm_bwd_noalloc(1, t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(),
                                     4, 12, None)
    assert rc == -21
