"""Symmetric device buffers: every rank allocates the same size with cudaMalloc, exports a CUDA IPC handle, and
maps every peer's allocation, so kernels can address any rank's copy with plain loads and stores over NVLink.

The handles travel over the existing process group (``all_gather_object``).  A buffer exposes its own memory as
a PyTorch tensor (zero-copy, via ``__cuda_array_interface__``) so that parameters' ``.grad`` views and bf16
compute copies can live directly inside communication memory.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

_DT = {torch.float32: ("<f4", 4), torch.bfloat16: ("<u2", 2), torch.int32: ("<i4", 4), torch.uint8: ("|u1", 1)}


class _RawCuda:
    def __init__(self, ptr: int, numel: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": None}


class SymmetricBuffer:
    def __init__(self, fabric, nbytes: int):
        from ..ops import cuda as K

        self._K = K
        self.rank, self.world = fabric.global_rank, fabric.world_size
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self.device = fabric.device
        ptr = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        K._check(K.lib.b200_ipc_alloc(C.c_longlong(self.nbytes), C.byref(ptr), handle), "ipc_alloc")
        self.own = ptr.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle))
        self.ptrs = []
        for q, h in enumerate(handles):
            if q == self.rank:
                self.ptrs.append(self.own)
            else:
                p = C.c_void_p()
                buf = (C.c_ubyte * 64).from_buffer_copy(h)
                K._check(K.lib.b200_ipc_open(buf, C.byref(p)), "ipc_open")
                self.ptrs.append(p.value)
        self._keep = []
        self.closed = False

    def ptr_array(self, byte_offset: int = 0):
        """ctypes array of N device pointers (own and peers) shifted by ``byte_offset``."""
        arr = (C.c_void_p * self.world)(*[p + byte_offset for p in self.ptrs])
        return arr

    def tensor(self, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        typestr, size = _DT[dtype]
        assert byte_offset + numel * size <= self.nbytes
        raw = _RawCuda(self.own + byte_offset, numel, typestr)
        t = torch.as_tensor(raw, device=self.device)
        if dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        self._keep.append(raw)
        return t

    def close(self) -> None:
        if self.closed:
            return
        self.closed = True
        torch.cuda.synchronize(self.device)
        for q, p in enumerate(self.ptrs):
            if q != self.rank:
                self._K.lib.b200_ipc_close(C.c_void_p(p))
        if dist.is_initialized():
            dist.barrier(device_ids=[self.device.index])  # nobody frees memory a peer still has mapped
        self._K.lib.b200_ipc_free(C.c_void_p(self.own))
