"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some callers cannot allocate device memory where they need this op (a plugin inside another
runtime's memory plan, a loop whose allocator is frozen). For them the library exports one entry
point whose scratch lives in the library's own device image. The test calls it twice in a row with
ctypes and compares with the regular entry point, which takes a caller-provided scratch buffer.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import forgeminds_b200
    path = os.path.join(os.path.dirname(forgeminds_b200.__file__), "_C.so")
    lib = ctypes.CDLL(path)
    fn = lib.fmb_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn


def test_matches_regular_entry_point_twice():
    from forgeminds_b200 import ops
    C = ops.require()
    fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # the third case needs more thread blocks than the built-in scratch has rows for (320): the grid is
    # clamped there and every block walks several row groups
    for seed, (rows, d) in enumerate([(777, 1024), (300, 4096), (16384, 512)]):
        g = torch.Generator(device="cuda").manual_seed(seed)
        x = torch.randn(rows, d, device="cuda", generator=g).to(torch.bfloat16)
        dy = torch.randn(rows, d, device="cuda", generator=g).to(torch.bfloat16)
        w = 1 + 0.1 * torch.randn(d, device="cuda", generator=g)
        _, rstd = C.rmsnorm_fwd(x, w, 1e-6)
        want_dx, want_dw = C.rmsnorm_bwd(dy, x, w, rstd, None, True)
        dx = torch.empty_like(x)
        dw = torch.empty(d, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, d, 0, 1,
                stream)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert torch.equal(dx, want_dx)
        assert torch.allclose(dw, want_dw, rtol=1e-4, atol=1e-4)     # the two sum the rows in different groupings


def test_refuses_rows_wider_than_the_scratch():
    fn = _lib()
    t = torch.zeros(8, 8192, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(8192, device="cuda")
    r = torch.ones(8, device="cuda")
    out = torch.empty_like(t)
    dw = torch.empty(8192, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), w.data_ptr(), r.data_ptr(), out.data_ptr(), dw.data_ptr(), 8, 8192, 0, 1,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -20


def test_refuses_a_width_the_kernels_cannot_vectorise():
    fn = _lib()
    t = torch.zeros(8, 36, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(36, device="cuda")
    r = torch.ones(8, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), w.data_ptr(), r.data_ptr(), t.data_ptr(), w.data_ptr(), 8, 36, 0, 1,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -22
