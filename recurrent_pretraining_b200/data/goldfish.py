"""Goldfish loss: deterministic token-loss dropout on the labels (recpre/utils.py:1395-1517).

Strategies: ``static`` (every k-th position), ``seeded_random``, ``hash-table`` (a fixed table of uniforms indexed by
the product of the previous ``context_width`` labels mod a prime) and ``hash-avalanche`` (Thomas Wang's 64-bit integer
hash of that product, truncated to 32 bits).  Dropped labels are replaced by ``ignore_index``.
"""
from __future__ import annotations

import torch

TABLE_SIZE = 1_000_003
_tables: dict = {}


def _hash_table(device) -> torch.Tensor:
    key = str(device)
    if key not in _tables:
        g = torch.Generator(device=device)
        g.manual_seed(2971215073)
        _tables[key] = torch.rand(TABLE_SIZE, device=device, generator=g)
    return _tables[key]


def hashint(key: torch.Tensor, width: int = 32) -> torch.Tensor:
    """Thomas Wang's 64-bit mix restricted to ``width`` bits, on int64 tensors with wrap-around arithmetic."""
    mask = (1 << width) - 1
    key = key.to(torch.int64)
    key = (~key + (key << 21)) & mask
    key = (key << 21) - key - 1
    key = key ^ (key >> 24)
    key = ((key + (key << 3)) + (key << 8)) & mask
    key = key * 265
    key = key ^ (key >> 14)
    key = ((key + (key << 2)) + (key << 4)) & mask
    key = key * 21
    key = key ^ (key >> 28)
    key = (key + (key << 31)) & mask
    return key


def apply_tld(labels: torch.Tensor, settings, ignore_index: int = -100):
    """Returns (masked labels, dropped-position indicator); ``labels`` itself is left untouched."""
    k, start, width = settings.k_token_loss_dropout, settings.start_position, settings.context_width
    strategy = settings.strategy
    out = labels.clone()
    B, S = labels.shape
    if strategy == "static":
        idx = torch.arange(S, device=labels.device)[start::k]
        out[:, idx] = ignore_index
        return out, idx
    if strategy in ("seeded_random", "pure_random"):
        drop = torch.randint(1, k + 1, labels.shape, device=labels.device) == k
        out[drop] = ignore_index
        return out, drop.int()
    keys = labels.unfold(1, width, 1).prod(dim=-1)
    if strategy == "hash-table":
        drop = _hash_table(labels.device)[keys % TABLE_SIZE] < 1.0 / k
    elif strategy == "hash-avalanche":
        drop = hashint(keys, 32) < ((1 << 32) - 1) / k
    else:
        raise NotImplementedError(f"{strategy} TLD strategy is not implemented. Try 'static' instead.")
    out[:, width - 1:][drop] = ignore_index
    return out, drop.int()
