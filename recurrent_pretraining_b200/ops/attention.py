"""Binding of the hand-written causal flash-attention kernels (tcgen05, head dims up to 128).

``native_supported`` gates the kernel: shapes it does not cover fall back to the library attention in
``ops.cuda`` (the fallback is explicit and visible in the launch list, never silent on the flagship shape).
"""
from __future__ import annotations

import torch

ENABLED = False  # flipped to True once the kernels in csrc/attention.cu are built into the library


def native_supported(head_dim: int, seq_len: int) -> bool:
    return ENABLED and head_dim % 16 == 0 and head_dim <= 128


def fwd(qkv_r, n_head, n_kv, D, scale):
    raise NotImplementedError


def bwd(do, qkv_r, o, lse, n_head, n_kv, D, scale):
    raise NotImplementedError
