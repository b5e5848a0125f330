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


def _aligned(n: int) -> int:
    return (n + ALIGN_ELEMS - 1) // ALIGN_ELEMS * ALIGN_ELEMS


def flatten_group(params, names, device, with_shadow: bool, hyper: dict, alloc=None) -> FlatGroup:
    """``alloc(kind, numel, dtype)`` may supply the three buffers (e.g. from symmetric communication memory)."""
    offsets, total = [], 0
    for p in params:
        offsets.append(total)
        total += _aligned(p.numel())
    total = max(total, ALIGN_ELEMS)
    if alloc is None:
        def alloc(kind, numel, dtype):
            return torch.zeros(numel, dtype=dtype, device=device)
    master = alloc("master", total, torch.float32)
    grad = alloc("grad", total, torch.float32)
    shadow = alloc("shadow", total, torch.bfloat16) if with_shadow else None
    for p, off in zip(params, offsets):
        n = p.numel()
        view = master[off:off + n].view(p.shape)
        view.copy_(p.detach().to(device=device, dtype=torch.float32))
        p.data = view
        p.grad = grad[off:off + n].view(p.shape)
        if with_shadow:
            lp = shadow[off:off + n].view(p.shape)
            lp.copy_(view)
            p._lp = lp
            p._fused_grad = True
    return FlatGroup(list(params), list(names), offsets, total, master, grad, shadow, dict(hyper))


def zero_grads(groups) -> None:
    for g in groups:
        g.grad.zero_()
