"""Activation checkpointing with selectively saved operator outputs (``activation_checkpoint_impl: sac | sac-attn |
sac%N``).

The reference builds these policies on torch's dispatcher-level selective checkpointing: keep the outputs of matrix
multiplications and attention, recompute everything else (recpre/config_dynamic.py:253-335); ``sac-attn`` keeps only
attention outputs; ``sac%N`` keeps every GEMM output except each N-th one.  The kernels here are launched through
``torch.autograd.Function``s that the dispatcher cannot see, so the same policies are applied one level up: while a
checkpointed region runs its first forward pass, every GEMM / attention op of ``ops.functional`` reports its output
to the region's ``SacRegion``; when the region is recomputed for backward, the op takes the kept output back instead of
launching its kernel (its autograd node still records the inputs, so backward is unchanged).  Norms, SwiGLU, RoPE and
the residual arithmetic -- a few percent of a block's time -- are what gets recomputed.

On CPU tensors the region falls back to plain recomputation of everything (torch's own selective contexts would work
there, but the CPU path exists for tests, not for memory savings).
"""
from __future__ import annotations

import threading
from contextlib import contextmanager
from functools import partial

import torch
import torch.utils.checkpoint

_tls = threading.local()


class SacRegion:
    """Bookkeeping of one checkpointed call: the outputs kept during the forward pass, replayed in call order."""

    def __init__(self, impl: str):
        self.keep_mm = impl.startswith("sac") and "sac-attn" not in impl
        self.keep_attn = impl.startswith("sac")
        self.every = 0
        if "sac%" in impl:
            self.every = int(impl.split("sac%")[1][0])
        self.kept: list = []
        self.mode = "off"
        self.cursor = 0
        self.mm_count = 0
        self.recomputed = 0     # kernels that had to run again (diagnostics / tests)

    def _wants(self, kind: str) -> bool:
        if kind == "attn":
            return self.keep_attn
        self.mm_count += 1
        if not self.keep_mm:
            return False
        return not (self.every and self.mm_count % self.every == 0)

    def record(self, kind: str, tensors):
        """Forward pass: called by an op after it produced ``tensors`` (a tuple)."""
        self.kept.append(tuple(t.detach() for t in tensors) if self._wants(kind) else None)

    def replay(self, kind: str):
        """Recomputation: the tuple kept for this call, or None when the op has to run again."""
        item = self.kept[self.cursor] if self.cursor < len(self.kept) else None
        self.cursor += 1
        if item is None:
            self.recomputed += 1
        return item


def current() -> SacRegion | None:
    r = getattr(_tls, "region", None)
    return r if r is not None and r.mode != "off" else None


def run_op(kind: str, compute):
    """``compute()`` -> tuple of tensors.  Inside a selective region the result is recorded (forward) or taken from the
    record (recomputation); outside it this is just ``compute()``."""
    r = current()
    if r is None:
        return compute()
    if r.mode == "forward":
        out = compute()
        r.record(kind, out)
        return out
    kept = r.replay(kind)
    return kept if kept is not None else compute()


@contextmanager
def _phase(region: SacRegion, mode: str):
    prev = getattr(_tls, "region", None)
    region.mode = mode
    if mode == "recompute":
        region.cursor = 0
    _tls.region = region
    try:
        yield
    finally:
        region.mode = "off"
        _tls.region = prev


def selective_checkpoint(fn, *args, impl: str = "sac", **kwargs):
    """Run ``fn(*args)`` under activation checkpointing with the policy named by ``impl``."""
    region = SacRegion(impl)

    def context_fn():
        return _phase(region, "forward"), _phase(region, "recompute")

    out = torch.utils.checkpoint.checkpoint(fn, *args, use_reentrant=False, preserve_rng_state=False,
                                            determinism_check="none", context_fn=context_fn, **kwargs)
    selective_checkpoint.last_region = region
    return out


def checkpoint_fn(impl: str):
    """The checkpoint callable for an ``activation_checkpoint_impl`` string (the counterpart of ``Config.checkpoint``):
    the placement words (per-block, per-iteration, in-coda) are read by the models, the policy word here."""
    if "sac%" in impl:
        return partial(selective_checkpoint, impl="sac%" + impl.split("sac%")[1][0])
    if "sac-attn" in impl:
        return partial(selective_checkpoint, impl="sac-attn")
    if "sac" in impl:
        return partial(selective_checkpoint, impl="sac")
    return partial(torch.utils.checkpoint.checkpoint, use_reentrant=False, preserve_rng_state=False,
                   determinism_check="none")
