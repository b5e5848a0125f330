"""Flat, bucket-friendly storage for parameters, gradients and optimizer state.

All parameters of one optimizer group live in one contiguous fp32 ``master`` buffer; gradients in a parallel
fp32 ``grad`` buffer (each ``p.grad`` is a permanent view, so wgrad GEMMs accumulate straight into the
communication buffer); the bf16 compute copies in a ``shadow`` buffer (``p._lp`` views) refreshed by the fused
optimizer kernel.  Tensor starts are aligned to 256 bytes so that TMA descriptors and 16-byte vector accesses
are always legal on every view.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

ALIGN_ELEMS = 128


@dataclass
class FlatGroup:
    params: list
    names: list
    offsets: list
    numel: int
    master: torch.Tensor
    grad: torch.Tensor
    shadow: torch.Tensor | None
    hyper: dict = field(default_factory=dict)
    state: dict = field(default_factory=dict)
    plan: object = None            # per-tensor ownership (parallel.segments.GroupShards) when the group is sharded
    master_sharded: bool = False   # ``master`` holds only this rank's pieces, concatenated in tensor order


def _aligned(n: int) -> int:
    return (n + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS


def flatten_group(params, names, device, with_shadow: bool, hyper: dict, alloc=None, shard=None) -> FlatGroup:
    """``alloc(kind, numel, dtype)`` may supply the buffers (e.g. from symmetric communication memory).

    ``shard = (world, rank)`` keeps only this rank's piece of every tensor in the fp32 ``master`` (parameter-sharded
    mode): the compute path reads the bf16 ``shadow`` only, ``p.data`` becomes a zero-stride placeholder of the right
    shape, and whole fp32 tensors are reassembled on demand (``parallel.p2p.ShardedStepper.full_master``)."""
    offsets, total = [], 0
    for p in params:
        offsets.append(total)
        total += _aligned(p.numel())
    total = max(total, ALIGN_ELEMS)
    if alloc is None:
        def alloc(kind, numel, dtype):
            return torch.zeros(numel, dtype=dtype, device=device)
    group = FlatGroup(list(params), list(names), offsets, total, None, None, None, dict(hyper))
    grad = alloc("grad", total, torch.float32)
    shadow = alloc("shadow", total, torch.bfloat16) if with_shadow else None
    if shard is not None:
        from .segments import GroupShards

        assert with_shadow, "sharded fp32 masters need the bf16 compute copies"
        world, rank = shard
        plan = GroupShards.plan(group, world)
        soff = plan.state_offsets(rank)
        master = torch.zeros(max(plan.owned(rank), 4), dtype=torch.float32, device=device)
        placeholder = torch.zeros(1, dtype=torch.float32, device=device)
        group.plan, group.master_sharded = plan, True
    else:
        master = alloc("master", total, torch.float32)
    for t, (p, off) in enumerate(zip(params, offsets)):
        n = p.numel()
        src = p.detach().to(device=device, dtype=torch.float32)
        if with_shadow:
            lp = shadow[off:off + n].view(p.shape)
            lp.copy_(src)
            p._lp = lp
            p._fused_grad = True
        if shard is not None:
            lo, hi = plan.local(t, rank)
            master[soff[t]:soff[t] + hi - lo].copy_(src.reshape(-1)[lo:hi])
            p.data = placeholder.expand(p.shape)
        else:
            view = master[off:off + n].view(p.shape)
            view.copy_(src)
            p.data = view
        p.grad = grad[off:off + n].view(p.shape)
    group.master, group.grad, group.shadow = master, grad, shadow
    return group


def zero_grads(groups) -> None:
    for g in groups:
        g.grad.zero_()
