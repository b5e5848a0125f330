"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some embedders of the kernel library may not call cudaMalloc (a host application owns all device memory, or an
allocator call is forbidden inside a latency-critical loop), so they cannot provide the scratch matrix the
regular entry point needs.  ``b200_rmsnorm_bwd_noalloc`` keeps that scratch in a fixed array inside the library.
This test checks it against the regular entry point on two consecutive calls (the array is shared and keeps the
previous call's contents, so the second call proves nothing stale leaks through) and checks the size limit.
The file name sorts last on purpose: a run that stops at the first failure has then executed every other test.
"""
import ctypes as C
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "recurrent_pretraining_b200", "_lib",
                   "libb200ops.so")


def _lib():
    lib = C.CDLL(LIB)
    fn = lib.b200_rmsnorm_bwd_noalloc
    fn.argtypes = [C.c_void_p] * 6 + [C.c_int, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    lib.b200_noalloc_last_error.restype = C.c_char_p
    return lib, fn


def _close(got, want, rtol, atol):
    err = (got.float() - want.float()).abs()
    tol = atol + rtol * want.float().abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g}"


def test_noalloc_matches_regular_entry_point_twice():
    from recurrent_pretraining_b200.ops import cuda as K

    lib, fn = _lib()
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (M, E) in enumerate([(300, 5280), (77, 480)]):  # second call: smaller problem over stale scratch
        x = torch.randn(M, E, device="cuda").bfloat16()
        dy = torch.randn(M, E, device="cuda").bfloat16()
        w = torch.rand(E, device="cuda") + 0.5
        _, rstd = K.rmsnorm_fwd(x, w, 1e-6)
        dx_ref, dw_ref = K.rmsnorm_bwd(dy, x, w, rstd)
        dx = torch.empty_like(x)
        dw = torch.empty(E, dtype=torch.float32, device="cuda")
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), M, E, stream)
        assert rc == 0, lib.b200_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref), f"call {call}: dx differs"
        _close(dw, dw_ref, 2e-2, 2e-2 * M ** 0.5)


def test_noalloc_rejects_oversize_rows():
    lib, fn = _lib()
    t = torch.zeros(8, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), 0, t.data_ptr(), t.data_ptr(), 0, 1, 8200, 0)
    assert rc == -1
    assert b"at most 8192" in lib.b200_noalloc_last_error()
    rc = fn(t.data_ptr(), t.data_ptr(), 0, t.data_ptr(), t.data_ptr(), 0, 1, 100, 0)
    assert rc == -1
