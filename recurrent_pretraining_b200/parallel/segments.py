"""Per-tensor ownership of the flat parameter / gradient / optimizer-state buffers.

Rank q owns elements ``[q * per, min(numel, (q + 1) * per))`` of every tensor of a flat optimizer group.  ``per`` is a
whole number of leading-dimension rows whenever that keeps 16-byte alignment, so a row-sharded weight can be gathered
by the GEMM that consumes it (``parallel/ag_gemm.py``); otherwise the tensor is cut flat into aligned pieces.  Because
every tensor is cut over all ranks, any set of whole tensors (a "bucket": the coda, the recurrent core, the prelude ...)
is balanced over the ranks, which is what lets buckets be reduced as soon as their gradients are complete.

The same description is handed to the kernels as a small by-value table (``csrc/comm_seg.cu: TensorTable``) and is used
on the host for the sharded optimizer state, checkpoints and the CPU/gloo emulation of the sharded step.

The reference shards only optimizer state, by whole tensors and with hard-coded rank rules (recpre/optim.py:168-178).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

MAX_TT = 48
ALIGN = 128


class TensorTableC(C.Structure):
    _fields_ = [("n", C.c_int), ("n_ranks", C.c_int), ("off", C.c_longlong * MAX_TT), ("numel", C.c_longlong * MAX_TT),
                ("per", C.c_longlong * MAX_TT), ("soff", C.c_longlong * MAX_TT), ("stat", C.c_int * MAX_TT)]


def per_rank_elems(numel: int, rows: int, world: int) -> int:
    """Elements of one tensor owned by each rank (the last owners may hold fewer, or nothing)."""
    if world <= 1:
        return numel
    if rows > 0 and numel % rows == 0:
        cols = numel // rows
        per = -(-rows // world) * cols
        if per % 8 == 0:
            return per
    per = -(-numel // world)
    return -(-per // ALIGN) * ALIGN


@dataclass
class GroupShards:
    """Ownership of one flat group: parallel lists over its tensors."""
    names: list
    offs: list
    numels: list
    rows: list
    pers: list
    world: int

    @classmethod
    def plan(cls, group, world: int) -> "GroupShards":
        rows = [p.shape[0] if p.dim() > 0 else 1 for p in group.params]
        numels = [p.numel() for p in group.params]
        pers = [per_rank_elems(n, r, world) for n, r in zip(numels, rows)]
        return cls(list(group.names), list(group.offsets), numels, rows, pers, world)

    def local(self, t: int, q: int) -> tuple[int, int]:
        """(lo, hi) of rank q inside tensor t."""
        lo = min(q * self.pers[t], self.numels[t])
        return lo, min(lo + self.pers[t], self.numels[t])

    def segment(self, t: int, q: int) -> tuple[int, int]:
        """(start, length) of rank q's piece of tensor t in the flat buffer."""
        lo, hi = self.local(t, q)
        return self.offs[t] + lo, hi - lo

    def state_offsets(self, q: int) -> list:
        out, acc = [], 0
        for t in range(len(self.offs)):
            out.append(acc)
            acc += self.segment(t, q)[1]
        return out

    def owned(self, q: int) -> int:
        return sum(self.segment(t, q)[1] for t in range(len(self.offs)))

    def rows_per_rank(self, t: int) -> int | None:
        """Rows of tensor t per rank when it is row-sharded (None for a flat cut)."""
        cols = self.numels[t] // max(self.rows[t], 1)
        if self.world > 1 and cols and self.pers[t] % cols == 0 and self.numels[t] % self.rows[t] == 0:
            return self.pers[t] // cols
        return None

    def tables(self, tensor_ids, rank: int, stat_base: int = 0) -> list:
        """ctypes tables (at most MAX_TT tensors each) for the kernels; ``stat`` numbers the tensors from
        ``stat_base`` in group order."""
        soff = self.state_offsets(rank)
        out = []
        ids = list(tensor_ids)
        for c0 in range(0, len(ids), MAX_TT):
            chunk = ids[c0:c0 + MAX_TT]
            tb = TensorTableC()
            tb.n, tb.n_ranks = len(chunk), self.world
            for i, t in enumerate(chunk):
                tb.off[i], tb.numel[i], tb.per[i], tb.soff[i] = self.offs[t], self.numels[t], self.pers[t], soff[t]
                tb.stat[i] = stat_base + t
            out.append(tb)
        return out


def bucket_of(name: str, group_kind: str, n_layer: int = 0, coarse: bool = False) -> str:
    """Readiness bucket of a parameter: one per prelude block and per coda block (``coarse``: one for all of them), one
    for the recurrent core with the adapter, ``upper`` for the top half of a plain GPT stack, ``last`` for the rest.
    The small fp32 group (norm scales, biases) always goes last: its gradients pass through autograd's accumulation
    nodes, whose position in the backward order is not pinned down."""
    if group_kind == "norm":
        return "last"
    for part in ("coda", "prelude"):
        tag = f".{part}."
        if tag in name:
            idx = name.split(tag)[1].split(".")[0]
            return f"{part}.{0 if coarse or not idx.isdigit() else int(idx)}"
    if ".core_block." in name or ".adapter." in name or "step_embedding" in name:
        return "core"
    if ".h." in name and n_layer > 1:
        try:
            idx = int(name.split(".h.")[1].split(".")[0])
        except ValueError:
            return "last"
        return "upper" if idx >= n_layer // 2 else "last"
    return "last"


def _split(bucket: str) -> tuple[str, int]:
    head, _, idx = bucket.partition(".")
    return head, int(idx) if idx.isdigit() else 0


def readiness_key(bucket: str) -> tuple:
    """Sort key: the order in which the buckets' gradients complete during backward (the coda's last block first, then
    down to its first block, the core, the prelude from its last block down, and the rest at the very end)."""
    head, idx = _split(bucket)
    return ({"coda": 0, "upper": 1, "core": 2, "prelude": 3}.get(head, 9), -idx)


def gather_key(bucket: str) -> tuple:
    """Sort key: the order in which the forward pass needs the buckets' weights."""
    head, idx = _split(bucket)
    return ({"last": 0, "prelude": 1, "upper": 2, "core": 3, "coda": 4}.get(head, 5), idx)


MAX_BUCKETS = 30
