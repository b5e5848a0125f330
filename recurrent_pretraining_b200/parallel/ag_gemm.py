"""All-gather fused into the consuming GEMM for row-sharded weights (ZeRO-3 style parameter sharding).

Each rank keeps 1/N of a weight's rows in symmetric (peer-mapped) memory.  ``GatheredWeight.gemm(x)`` runs ONE kernel
(``b200_ag_gemm``) in which copier warps pull the other ranks' shards over NVLink into a local full-size buffer, N-tile
by N-tile starting with the local shard, while the tensor-core warps multiply the tiles that have landed.  Afterwards the
local buffer holds the whole weight, so the other recurrences of the same step use the plain GEMM on it: the gather is
paid once per step and hidden behind the first use.

The reference has no counterpart (its only sharding is the optimizer-state ZeRO-1 wrapper, recpre/optim.py:131-263).
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import cuda as K
from .symm import SymmetricBuffer

_vp, _i = C.c_void_p, C.c_int
_ag = K._sig("b200_ag_gemm", [_vp, _vp, _vp, _vp, _vp] + [_i] * 9 + [_vp, _vp])


class GatheredWeight:
    def __init__(self, fabric, n_rows: int, n_cols: int):
        assert n_cols % 8 == 0
        self.fabric = fabric
        self.rank, self.world = fabric.global_rank, fabric.world_size
        self.N, self.K = n_rows, n_cols
        self.rows_per_shard = (n_rows + self.world - 1) // self.world
        self.buf = SymmetricBuffer(fabric, self.rows_per_shard * n_cols * 2)
        self.shard = self.buf.tensor(torch.bfloat16, self.rows_per_shard * n_cols).view(self.rows_per_shard, n_cols)
        self.full = torch.empty(n_rows, n_cols, dtype=torch.bfloat16, device=fabric.device)
        self.done = torch.zeros((n_rows + 239) // 240 + 1, dtype=torch.int32, device=fabric.device)
        self.gathered = False

    @property
    def my_rows(self) -> slice:
        lo = self.rank * self.rows_per_shard
        return slice(lo, min(lo + self.rows_per_shard, self.N))

    def load_full(self, w: torch.Tensor) -> None:
        """Keep this rank's rows of a full weight (tests / initialisation)."""
        rows = self.my_rows
        self.shard[: rows.stop - rows.start].copy_(w[rows].to(torch.bfloat16))
        self.gathered = False

    def gemm(self, x: torch.Tensor) -> torch.Tensor:
        """y = x W^T.  The first call after the shards changed gathers while it multiplies; the caller must have made
        sure (a barrier after the step that wrote the shards) that every rank's shard is complete."""
        x2 = x.reshape(-1, x.shape[-1])
        if self.gathered or x2.shape[0] < 256:
            if not self.gathered:
                self.gather_only()
            return K.gemm_nt(x2, self.full).view(*x.shape[:-1], self.N)
        assert x2.dtype == torch.bfloat16 and x2.stride(1) == 1
        y = torch.empty(x2.shape[0], self.N, dtype=torch.bfloat16, device=x.device)
        K._check(_ag(x2.data_ptr(), C.cast(self.buf.ptr_array(), C.c_void_p), self.full.data_ptr(), y.data_ptr(),
                     self.done.data_ptr(), x2.shape[0], self.N, self.K, x2.stride(0), self.N, self.world, self.rank,
                     self.rows_per_shard, 0, K._stream(), K.err_word(x.device).data_ptr()), "ag_gemm")
        self.gathered = True
        return y.view(*x.shape[:-1], self.N)

    def gather_only(self) -> None:
        """Plain gather through the library (used for tiny inputs and as the baseline of the benchmark)."""
        import torch.distributed as dist

        parts = [torch.empty_like(self.shard) for _ in range(self.world)]
        dist.all_gather(parts, self.shard.contiguous())
        self.full.copy_(torch.cat(parts, 0)[: self.N])
        self.gathered = True

    def invalidate(self) -> None:
        self.gathered = False

    def close(self) -> None:
        self.buf.close()
