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
        # and against the plain fp32 statement of the op
        x32 = x.float().requires_grad_(True)
        w32 = w.clone().requires_grad_(True)
        y = (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16).float() * w32
        y.backward(dy.float())
        _close(dx, x32.grad, 3e-2, 3e-2)
        _close(dw, w32.grad, 2e-2, 2e-2 * M ** 0.5)


def test_noalloc_rejects_oversize_rows():
    lib, fn = _lib()
    t = torch.zeros(8, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), 0, t.data_ptr(), t.data_ptr(), 0, 1, 8200, 0)
    assert rc == -1
    assert b"at most 8192" in lib.b200_noalloc_last_error()
    rc = fn(t.data_ptr(), t.data_ptr(), 0, t.data_ptr(), t.data_ptr(), 0, 1, 100, 0)
    assert rc == -1


def test_noalloc_rejects_bad_pointers_before_any_launch():
    """A NULL or misaligned buffer is refused on the host (rc -1, nothing launched), because on the device it would be
    a fault that costs the embedding application its CUDA context."""
    from recurrent_pretraining_b200.ops import cuda as K

    lib, fn = _lib()
    M, E = 4, 64
    x = torch.randn(M, E + 8, device="cuda").bfloat16()
    dy = torch.randn(M, E, device="cuda").bfloat16()
    rstd = torch.ones(M, device="cuda")
    dx = torch.full((M, E), 7.0, device="cuda").bfloat16()
    torch.cuda.synchronize()
    before = K.launch_count()
    rc = fn(dy.data_ptr(), x.data_ptr(), 0, rstd.data_ptr(), 0, 0, M, E, 0)           # dx == NULL
    assert rc == -1 and b"NULL" in lib.b200_noalloc_last_error()
    rc = fn(dy.data_ptr(), x.data_ptr() + 2, 0, rstd.data_ptr(), dx.data_ptr(), 0, M, E, 0)   # x off by one element
    assert rc == -1 and b"16-byte" in lib.b200_noalloc_last_error()
    torch.cuda.synchronize()
    assert K.launch_count() == before
    assert bool((dx.float() == 7.0).all())      # the output was never touched
