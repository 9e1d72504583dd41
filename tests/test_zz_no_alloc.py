"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some callers of the operator library cannot allocate device memory: a process that gave
the whole GPU to its own memory pool, or a runtime that forbids the device-wide
synchronisation cudaMalloc implies.  For them the library exports
``tb200_rmsnorm_bwd_noalloc`` whose scratch buffer is a static device array.  This test
calls the symbol with raw pointers (ctypes, no torch operator involved) twice in a row
and checks both results against the regular allocating operator.  It lives in the last
collected file so a failure here cannot hide the result of any other test.
"""

import ctypes

import pytest
import torch

from torchtitan_b200.ops import ext

pytestmark = pytest.mark.gpu


def _lib():
    assert ext.load(), "the sm_100a extension must be built in-tree"
    lib = ctypes.CDLL(ext.LIB_PATH)
    fn = lib.tb200_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.tb200_noalloc_strerror.restype = ctypes.c_char_p
    lib.tb200_noalloc_strerror.argtypes = [ctypes.c_int]
    return lib


def _call(lib, dy, x, w, rstd, dx, dw):
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.tb200_rmsnorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                       dw.data_ptr(), x.shape[0], x.shape[1], 0 if x.dtype == torch.bfloat16 else 1,
                                       ctypes.c_void_p(stream))
    assert rc == 0, lib.tb200_noalloc_strerror(rc).decode()


@pytest.mark.parametrize("dtype,rows,dim", [(torch.bfloat16, 1000, 4096), (torch.float32, 37, 1024),
                                            (torch.bfloat16, 3, 8192), (torch.float32, 129, 8192)])
def test_noalloc_matches_allocating_operator_twice(dtype, rows, dim):
    lib = _lib()
    torch.manual_seed(0)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    for call in range(2):  # the second call reuses the scratch left by the first
        x = torch.randn(rows, dim, device="cuda", dtype=dtype)
        w = (torch.rand(dim, device="cuda") + 0.5).to(dtype)
        dy = torch.randn(rows, dim, device="cuda", dtype=dtype) * (call + 1)
        _, rstd = torch.ops.tb200.rmsnorm_fwd(x, w, 1e-5)
        dx_ref, dw_ref = torch.ops.tb200.rmsnorm_bwd(dy, x, w, rstd)
        dx = torch.empty_like(x)
        dw = torch.empty(dim, device="cuda", dtype=torch.float32)
        before = torch.cuda.memory_allocated()
        _call(lib, dy, x, w, rstd, dx, dw)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.allclose(dx.float(), dx_ref.float(), atol=tol, rtol=tol)
        assert torch.allclose(dw, dw_ref, atol=1e-2 * rows ** 0.5 if dtype == torch.bfloat16 else 1e-3, rtol=1e-3)


def test_noalloc_with_no_rows_writes_a_zero_weight_gradient():
    lib = _lib()
    dim = 2048
    x = torch.ones(1, dim, device="cuda", dtype=torch.bfloat16)   # valid pointers; zero rows are passed below
    w = torch.ones(dim, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(1, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        dw = torch.full((dim,), 7.0, device="cuda")
        rc = lib.tb200_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), x.data_ptr(),
                                           dw.data_ptr(), 0, dim, 0, ctypes.c_void_p(stream))
        assert rc == 0, lib.tb200_noalloc_strerror(rc).decode()
        torch.cuda.synchronize()
        assert float(dw.abs().max()) == 0.0


def test_noalloc_rejects_rows_longer_than_the_static_scratch():
    lib = _lib()
    x = torch.zeros(2, 16384, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(16384, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(2, device="cuda")
    dw = torch.zeros(16384, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.tb200_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), x.data_ptr(),
                                       dw.data_ptr(), 2, 16384, 0, ctypes.c_void_p(stream))
    assert rc == 1
    assert b"8192" in lib.tb200_noalloc_strerror(rc)
    rc = lib.tb200_rmsnorm_bwd_noalloc(x.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), x.data_ptr(),
                                       dw.data_ptr(), 2, 100, 0, ctypes.c_void_p(stream))
    assert rc == 2
