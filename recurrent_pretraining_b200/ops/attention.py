"""Binding of the hand-written causal flash-attention kernels (tcgen05 MMAs, S/P/O tiles in tensor memory).

Forward and backward operate on the packed, already rotated qkv tensor [B, S, (H + 2 Hkv) * D]; head dims 64, 96 and
128 are built.  Other head dims use the library attention in ``ops.cuda`` (visible in the launch list).
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import cuda as K

_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
_fwd = K._sig("b200_attn_fwd", [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp])
_bwd = K._sig("b200_attn_bwd", [_vp] * 7 + [_i] * 5 + [_f, _vp, _vp]) if hasattr(K.lib, "b200_attn_bwd") else None

_set_variant = K._sig("b200_attn_set_fwd_variant", [_i])


def set_fwd_variant(v: int) -> int:
    """1: one query tile per CTA (P through shared memory); 2: two query tiles per CTA, P in tensor memory (default).
    Returns the previous setting."""
    return int(_set_variant(int(v)))


_set_bwd_variant = K._sig("b200_attn_set_bwd_variant", [_i])


def set_bwd_variant(v: int) -> int:
    """1: query-major tiles (P and dS through shared memory); 2: transposed tiles with P^T / dS^T in tensor memory
    (default).  Returns the previous setting."""
    return int(_set_bwd_variant(int(v)))


# Training runs on the native kernels (B200_NATIVE_ATTENTION=0 selects the library SDPA instead).  Measured on the
# flagship shape (B=1, S=4096, 55 heads of 96): native forward 0.222 ms / backward 0.99 ms, library forward 0.18 ms /
# forward-recompute + backward + copies 1.15-1.24 ms; the whole training step is the same either way (728.8 vs 728.9 ms).
ENABLED = os.environ.get("B200_NATIVE_ATTENTION", "1") == "1"
NATIVE_BWD = _bwd is not None and os.environ.get("B200_NATIVE_ATTENTION_BWD", "1") == "1"


PREFILL = os.environ.get("B200_NATIVE_PREFILL", "1") == "1"


def native_prefill_supported(head_dim: int) -> bool:
    """Inference prefill (fresh sequence, forward only) runs on the native kernel: no library call sits between the
    decode engine and its KV cache."""
    return PREFILL and head_dim in (64, 96, 128)


def native_supported(head_dim: int, seq_len: int) -> bool:
    return ENABLED and head_dim in (64, 96, 128)


def fwd(qkv_r, n_head, n_kv, D, scale):
    B, S, W = qkv_r.shape
    assert qkv_r.is_contiguous() and qkv_r.dtype == torch.bfloat16
    o = torch.empty(B, S, n_head * D, dtype=torch.bfloat16, device=qkv_r.device)
    lse = torch.empty(B, n_head, S, dtype=torch.float32, device=qkv_r.device)
    K._check(_fwd(qkv_r.data_ptr(), o.data_ptr(), lse.data_ptr(), B, S, n_head, n_kv, D, float(scale), K._stream(),
                  K.err_word(qkv_r.device).data_ptr()), "attn_fwd")
    return o, lse


def bwd(do, qkv_r, o, lse, n_head, n_kv, D, scale):
    """Gradient with respect to the packed rotated qkv tensor."""
    B, S, W = qkv_r.shape
    if not NATIVE_BWD:
        return K._attention_bwd_library(do, qkv_r, n_head, n_kv, D, scale)
    do = do.contiguous()
    assert do.dtype == torch.bfloat16 and o.is_contiguous() and qkv_r.is_contiguous()
    dqkv = torch.empty_like(qkv_r)
    # fp32 dQ accumulator, padded to whole 128-query blocks (the v2 kernel keeps it block-interleaved)
    dq_acc = torch.zeros(B * n_head * ((S + 127) // 128) * 128 * D, dtype=torch.float32, device=qkv_r.device)
    delta = torch.empty(B, n_head, S, dtype=torch.float32, device=qkv_r.device)
    K._check(_bwd(qkv_r.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(),
                  dqkv.data_ptr(), B, S, n_head, n_kv, D, float(scale), K._stream(),
                  K.err_word(qkv_r.device).data_ptr()), "attn_bwd")
    return dqkv
