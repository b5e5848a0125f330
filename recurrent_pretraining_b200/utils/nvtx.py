"""NVTX ranges around the phases of a training step (forward: prelude / recurrence / coda / loss, backward, gradient
reduction and update, parameter gathers), for timeline tools.  Off unless ``B200_NVTX=1``: a disabled range costs one
attribute test.  The reference has no profiler integration of its own (only wall-clock step timing, train.py:496-498)."""
from __future__ import annotations

import os
from contextlib import contextmanager

ENABLED = os.environ.get("B200_NVTX", "0") == "1"
_names: list = []          # ranges opened since the last reset, in order (tests look at this)


def enable(on: bool = True) -> None:
    global ENABLED
    ENABLED = bool(on)


@contextmanager
def range(name: str):  # noqa: A001
    if not ENABLED:
        yield
        return
    import torch

    pushed = False
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        pushed = True
    _names.append(name)
    try:
        yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()


def opened() -> list:
    return list(_names)


def reset() -> None:
    _names.clear()
