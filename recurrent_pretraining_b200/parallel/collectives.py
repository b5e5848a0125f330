"""One-launch NVLink collectives on bf16 gradient buckets (``csrc/comm_fused.cu``): all-reduce (one-pass "two-shot":
every rank reduces its slice and stores the result into all ranks), one-shot all-reduce for small buckets,
reduce-scatter, push all-gather, and reduce-scatter followed by a clipped AdamW on the slice that pushes the new bf16
parameters -- each fused with the bf16 -> fp32 cast, a scale and the squared-norm partial, with the cross-rank
handshakes inside the data kernel.

This is the bucket-level form of what the training step does on the flat gradient (``parallel/p2p.py``); it exists for
the communication sweep (``utils/comm_bench.py``) and for callers that reduce individual buckets.  The reference's
counterpart is the chunked NCCL all-reduce of recpre/utils.py:1013-1043.
"""
from __future__ import annotations

import ctypes as C

import torch

from .symm import SymmetricBuffer

ONE_SHOT_MAX_BYTES = 2 << 20     # below this the one-shot form (no stores to peers, one handshake) is faster


class FusedCollectives:
    def __init__(self, fabric, max_elems: int, timeout_ms: int = 20000):
        from ..ops import cuda as K

        self.K, self.fabric = K, fabric
        self.rank, self.N, self.dev = fabric.global_rank, fabric.world_size, fabric.device
        self.max_elems = (max_elems + 8 * self.N - 1) // (8 * self.N) * (8 * self.N)
        self.inp = SymmetricBuffer(fabric, self.max_elems * 2)        # bf16 bucket of every rank
        self.out = SymmetricBuffer(fabric, self.max_elems * 4)        # fp32 result of every rank
        self.ctrl = SymmetricBuffer(fabric, 1024)                     # slot A at 0, slot B at 64, norm partial at 128
        self.bucket = self.inp.tensor(torch.bfloat16, self.max_elems)
        self.result = self.out.tensor(torch.float32, self.max_elems)
        self.partial = self.ctrl.tensor(torch.float32, 1, 128)
        self.slot_a, self.slot_b = self.ctrl.ptr_array(0), self.ctrl.ptr_array(64)
        self.partial_ptrs = self.ctrl.ptr_array(128)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.gnorm = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.err = K.err_word(self.dev)
        self.timeout_ms = timeout_ms
        self.epoch = 0
        self.in_ptrs, self.out_ptrs = self.inp.ptr_array(), self.out.ptr_array()

    def slice_elems(self, count: int) -> int:
        per = (count + self.N - 1) // self.N
        return (per + 7) // 8 * 8

    def my_slice(self, count: int) -> tuple[int, int]:
        per = self.slice_elems(count)
        lo = min(self.rank * per, count)
        return lo, min(lo + per, count)

    def _hs(self):
        self.epoch += 1
        return (self.slot_a, self.slot_b, C.c_void_p(self.ticket.data_ptr()), C.c_uint(self.epoch), self.timeout_ms)

    def _reduce(self, count: int, mode: int, scale: float, with_norm: bool, ctas: int = 0) -> None:
        K = self.K
        assert count % 8 == 0 and count <= self.max_elems
        if with_norm:
            self.partial.zero_()
        a, b, ticket, epoch, to = self._hs()
        K._check(K.lib.b200_allreduce_bf16_fused(
            self.in_ptrs, self.out_ptrs, self.rank, self.N, C.c_longlong(self.slice_elems(count)), C.c_longlong(count),
            C.c_float(scale), C.c_void_p(self.partial.data_ptr() if with_norm else 0), mode, a, b, ticket, epoch, to,
            ctas, C.c_void_p(self.err.data_ptr()), C.c_void_p(K._stream())), "allreduce_bf16_fused")

    def all_reduce(self, count: int, scale: float = 1.0, with_norm: bool = True, one_shot: bool | None = None,
                   ctas: int = 0) -> torch.Tensor:
        """fp32 ``scale * sum over ranks`` of the first ``count`` elements of every rank's bucket, on every rank.
        With the one-shot form ``partial`` holds the squared norm of the WHOLE result (the same on every rank); with the
        sliced form it holds this rank's slice's share."""
        if one_shot is None:
            one_shot = count * 2 <= ONE_SHOT_MAX_BYTES
        self._reduce(count, 2 if one_shot else 0, scale, with_norm, ctas)
        return self.result[:count]

    def reduce_scatter(self, count: int, scale: float = 1.0, with_norm: bool = True, ctas: int = 0) -> torch.Tensor:
        """This rank's slice of the reduced bucket (fp32 view into ``result``)."""
        self._reduce(count, 1, scale, with_norm, ctas)
        lo, hi = self.my_slice(count)
        return self.result[lo:hi]

    def all_gather_bf16(self, count: int, ctas: int = 0) -> torch.Tensor:
        """Every rank's slice of its own bucket is stored into all peers' buckets (in place)."""
        K = self.K
        a, b, ticket, epoch, to = self._hs()
        K._check(K.lib.b200_allgather_push_fused(self.in_ptrs, self.rank, self.N,
                                                 C.c_longlong(self.slice_elems(count) * 2), C.c_longlong(count * 2),
                                                 a, b, ticket, epoch, to, ctas, C.c_void_p(self.err.data_ptr()),
                                                 C.c_void_p(K._stream())), "allgather_push_fused")
        return self.bucket[:count]

    def reduce_scatter_adamw(self, count: int, p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, shadow: SymmetricBuffer,
                             *, lr: float, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1, step: int = 1,
                             max_norm: float = 1.0, scale: float = 1.0) -> torch.Tensor:
        """Reduce-scatter of the bucket (cast, scale, norm partial), then -- second launch -- global-norm clip and AdamW
        on this rank's slice (``p``, ``m``, ``v``: fp32 arrays of the slice) whose new bf16 values are stored into every
        rank's ``shadow`` buffer at the slice's offset.  Returns the global gradient norm (device scalar)."""
        K = self.K
        g = self.reduce_scatter(count, scale, with_norm=True)
        lo, hi = self.my_slice(count)
        if hi > lo:
            assert p.numel() == hi - lo
        a, b, ticket, epoch, to = self._hs()
        b1, b2 = betas
        K._check(K.lib.b200_adamw_slice_push(
            C.c_void_p(p.data_ptr()), C.c_void_p(g.data_ptr()), C.c_void_p(m.data_ptr()), C.c_void_p(v.data_ptr()),
            C.c_longlong(hi - lo), C.c_longlong(lo), shadow.ptr_array(), self.partial_ptrs, self.rank, self.N,
            C.c_float(lr), C.c_float(b1), C.c_float(b2), C.c_float(eps), C.c_float(weight_decay),
            C.c_float(1 - b1 ** step), C.c_float(1 - b2 ** step), C.c_float(max_norm),
            C.c_void_p(self.gnorm.data_ptr()), a, b, ticket, epoch, to, C.c_void_p(self.err.data_ptr()),
            C.c_void_p(K._stream())), "adamw_slice_push")
        return self.gnorm

    def close(self) -> None:
        torch.cuda.synchronize(self.dev)
        for buf in (self.inp, self.out, self.ctrl):
            buf.close()
