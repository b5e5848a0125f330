"""Data-parallel gradient synchronisation with hand-written NVLink kernels on symmetric memory.

One optimizer step runs, on the training stream and without host synchronisation:

    barrier -> reduce-scatter of every flat fp32 gradient buffer (each rank sums its 1/N slice from all peers and
    accumulates the squared norm of the result) -> barrier that also exchanges the N norm partials -> AdamW on the
    owned slice only (optimizer state is sharded 1/N), whose epilogue pushes the updated bf16 compute copy to every
    rank -> barrier

This replaces the reference's post-backward chunked fp32 all-reduce followed by a replicated clip and a replicated
(or ZeRO-1 broadcast) optimizer step (recpre/utils.py:1004-1043,1196-1206; recpre/optim.py:131-263).  NVLink traffic per
GPU and step is (N-1)/N * (4 + 2) bytes per parameter instead of 2 * (N-1)/N * 4 for a two-shot fp32 all-reduce
(plus 4 bytes per parameter of ZeRO-1 broadcasts in the reference's production setting).

fp32 master weights of non-owned slices go stale by design; ``gather_master`` refreshes them (checkpointing).
The tiny norm/bias group is consumed in fp32 by the kernels, so its master values are pushed as well.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .symm import SymmetricBuffer

ALIGN = 128


def shard_range(numel: int, rank: int, world: int) -> tuple[int, int]:
    per = (numel + world - 1) // world
    per = (per + ALIGN - 1) // ALIGN * ALIGN
    lo = min(rank * per, numel)
    return lo, min(lo + per, numel)


class P2PAllocator:
    """Hands out flat buffers that live in symmetric memory; remembers them per (group index, kind)."""

    def __init__(self, fabric):
        self.fabric = fabric
        self.buffers: dict = {}

    def __call__(self, group_index: int, kind: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        size = 4 if dtype == torch.float32 else 2
        buf = SymmetricBuffer(self.fabric, numel * size)
        self.buffers[(group_index, kind)] = buf
        return buf.tensor(dtype, numel)


class P2PReducer:
    def __init__(self, fabric, groups, allocator: P2PAllocator, timeout_ms: int = 20000):
        from ..ops import cuda as K

        self.K, self.fabric, self.groups, self.alloc = K, fabric, groups, allocator
        self.rank, self.world = fabric.global_rank, fabric.world_size
        self.timeout_ms = timeout_ms
        self.epoch = 0
        # control block: N flags (uint32) + one float (norm partial) at byte 256
        self.ctrl = SymmetricBuffer(fabric, 512)
        self.flag_ptrs = self.ctrl.ptr_array(0)
        self.partial_ptrs = self.ctrl.ptr_array(256)
        self.partial = self.ctrl.tensor(torch.float32, 1, 256)
        self.ranges = [shard_range(g.numel, self.rank, self.world) for g in groups]
        self.grad_ptrs = [allocator.buffers[(i, "grad")].ptr_array() for i in range(len(groups))]
        self.shadow_ptrs = [allocator.buffers[(i, "shadow")].ptr_array() for i in range(len(groups))]
        self.master_ptrs = [allocator.buffers[(i, "master")].ptr_array() for i in range(len(groups))]
        dist.barrier(device_ids=[fabric.device.index])

    # ------------------------------------------------------------------------------------------
    def _barrier(self, with_norm_into=None) -> None:
        K = self.K
        self.epoch += 1
        total = with_norm_into.data_ptr() if with_norm_into is not None else 0
        K._check(K.lib.b200_barrier(self.flag_ptrs, self.rank, self.world, C.c_uint(self.epoch), self.timeout_ms,
                                    self.partial_ptrs if with_norm_into is not None else None, C.c_void_p(total),
                                    C.c_void_p(K.err_word(self.fabric.device).data_ptr()), C.c_void_p(K._stream())),
                 "barrier")

    def begin_backward(self, model, accumulating: bool) -> None:
        pass

    def step(self, optimizer, max_norm: float, grad_scale: float, do_update: bool) -> None:
        """Reduce, clip and update (see module docstring).  ``optimizer`` is a sharded ``FusedAdamW``."""
        K = self.K
        st = C.c_void_p(K._stream())
        self._barrier()
        self.partial.zero_()
        for gi, g in enumerate(self.groups):
            lo, hi = self.ranges[gi]
            K._check(K.lib.b200_reduce_scatter_f32(self.grad_ptrs[gi], self.rank, self.world, C.c_longlong(lo),
                                                   C.c_longlong(hi - lo), C.c_void_p(self.partial.data_ptr()), 0, st),
                     "reduce_scatter")
        self._barrier(with_norm_into=optimizer.gnorm_sq)
        optimizer.step_count += 1 if do_update else 0
        for gi, (g, h) in enumerate(zip(self.groups, optimizer.param_groups)):
            lo, hi = self.ranges[gi]
            if lo > 0:
                g.grad[:lo].zero_()
            if hi < g.numel:
                g.grad[hi:].zero_()
            if hi <= lo:
                continue
            if not do_update:
                g.grad[lo:hi].zero_()
                continue
            b1, b2 = h["betas"]
            t = optimizer.step_count
            push_master = gi == len(self.groups) - 1  # the norm / bias group is read in fp32 by the kernels
            K._check(K.lib.b200_adamw_push(
                C.c_void_p(g.master.data_ptr()), C.c_void_p(g.grad.data_ptr()),
                C.c_void_p(g.state["m"].data_ptr()), C.c_void_p(g.state["v"].data_ptr()), self.shadow_ptrs[gi],
                self.master_ptrs[gi] if push_master else None, self.world, C.c_longlong(lo), C.c_longlong(hi - lo),
                C.c_void_p(optimizer.gnorm_sq.data_ptr()), C.c_float(float(h["lr"])), C.c_float(b1), C.c_float(b2),
                C.c_float(h["eps"]), C.c_float(h["weight_decay"]), C.c_float(1.0 - b1 ** t), C.c_float(1.0 - b2 ** t),
                C.c_float(max_norm), C.c_float(grad_scale), 1, int(optimizer.atan2), st), "adamw_push")
        self._barrier()

    @torch.no_grad()
    def gather_master(self) -> None:
        """Make every rank's fp32 master copy complete (owners broadcast their slices over NCCL)."""
        for gi, g in enumerate(self.groups):
            for q in range(self.world):
                lo, hi = shard_range(g.numel, q, self.world)
                if hi > lo:
                    dist.broadcast(g.master[lo:hi], src=q)

    def close(self) -> None:
        torch.cuda.synchronize(self.fabric.device)
        self.ctrl.close()
        for buf in self.alloc.buffers.values():
            buf.close()
