"""Other formulations of rotary position embedding, kept as cross-checks of the one the models use
(``ops.reference.rope_interleaved``: rotate the pairs (2i, 2i+1) by angle pos * base^(-2i/d)).

The reference keeps a similar collection (recpre/misc.py:1-65).  Three views of the same rotation:

* ``rope_complex``      treat each pair as a complex number and multiply by exp(i * angle) -- identical to the
  interleaved form up to rounding;
* ``rope_rotate_half``  the GPT-NeoX layout: the pair is (channel j, channel j + d/2).  It equals the interleaved form
  on a channel-permuted tensor (``to_half_layout`` / ``from_half_layout`` are the permutations), which is what a
  checkpoint converter between the two conventions has to apply to the q/k projection rows;
* ``rope_matrix``       the explicit block-diagonal rotation matrix per position (tiny shapes; tests only).
"""
from __future__ import annotations

import torch


def angles(head_dim: int, length: int, base: float = 50000.0, condense: int = 1) -> torch.Tensor:
    """[length, head_dim / 2] rotation angles in fp32."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    return torch.outer(torch.arange(length, dtype=torch.float32) / condense, inv)


def complex_table(head_dim: int, length: int, base: float = 50000.0) -> torch.Tensor:
    a = angles(head_dim, length, base)
    return torch.polar(torch.ones_like(a), a)


def rope_complex(x: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x [B, S, H, D]; table complex [S, D/2]."""
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2).contiguous())
    out = torch.view_as_real(xc * table[None, :, None, :]).flatten(-2)
    return out.to(x.dtype)


def to_half_layout(x: torch.Tensor) -> torch.Tensor:
    """Interleaved pairs (2i, 2i+1) -> NeoX halves (i, i + D/2)."""
    return torch.cat([x[..., 0::2], x[..., 1::2]], dim=-1)


def from_half_layout(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return torch.stack([x[..., :d], x[..., d:]], dim=-1).flatten(-2)


def rope_rotate_half(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """NeoX form on a half-layout tensor: x * cos + rotate_half(x) * sin with the tables repeated over both halves."""
    d = x.shape[-1] // 2
    cos = torch.cat([ang.cos(), ang.cos()], dim=-1)[None, :, None, :]
    sin = torch.cat([ang.sin(), ang.sin()], dim=-1)[None, :, None, :]
    xf = x.float()
    rot = torch.cat([-xf[..., d:], xf[..., :d]], dim=-1)
    return (xf * cos + rot * sin).to(x.dtype)


def rope_matrix(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
    """Explicit rotation matrices (interleaved layout); O(D^2) per position."""
    S, half = ang.shape
    R = torch.zeros(S, 2 * half, 2 * half)
    idx = torch.arange(half)
    c, s = ang.cos(), ang.sin()
    R[:, 2 * idx, 2 * idx] = c
    R[:, 2 * idx, 2 * idx + 1] = -s
    R[:, 2 * idx + 1, 2 * idx] = s
    R[:, 2 * idx + 1, 2 * idx + 1] = c
    return torch.einsum("sde,bshe->bshd", R, x.float()).to(x.dtype)
