"""Goldfish loss: deterministic token-loss dropout on the labels (recpre/utils.py:1395-1517).

Strategies: ``static`` (every k-th position), ``seeded_random`` / ``pure_random`` (each position with probability 1/k
from the global / a time-seeded generator), ``random_but_consisent_for_given_micro_batch`` (generator seeded by the sum
of the labels), ``hash-table`` (a fixed table of uniforms indexed by the product of the previous ``context_width``
labels mod a prime), ``hash-avalanche`` (Thomas Wang's 64-bit integer hash of that product, truncated to 32 bits) and
``hash-legacy`` (one generator draw per position, seeded by the product; slow, for cross-checks).  Dropped labels are
replaced by ``ignore_index``.

The random strategies and ``hash-legacy`` apply their 0/1 draw as a boolean mask over positions.  The reference indexes
with the 0/1 integers instead (recpre/utils.py:1450-1480), which blanks rows 0 and 1 of the batch whatever was drawn,
and its ``hash-legacy`` never hands its seeded generator to the draw; the hash strategies that the shipped runs use
(``hash-table``, ``hash-avalanche``) and ``static`` are the same in both.
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
    if strategy in ("seeded_random", "pure_random", "random_but_consisent_for_given_micro_batch"):
        gen = None
        if strategy == "pure_random":
            import time

            gen = torch.Generator().manual_seed(int(time.time()))
        elif strategy != "seeded_random":
            gen = torch.Generator().manual_seed(int(labels.sum().item()))
        drop = (torch.randint(1, k + 1, labels.shape, generator=gen) == k).to(labels.device)
        out[drop] = ignore_index
        return out, drop.int()
    if strategy == "hash-legacy":
        drop = torch.zeros(B, S, dtype=torch.bool)
        gen = torch.Generator()
        host = labels.cpu()
        for b in range(B):
            for pos in range(width, S):
                gen.manual_seed(int(host[b, pos - width:pos].prod().item()) % (2 ** 63 - 1))
                drop[b, pos] = bool(torch.rand((1,), generator=gen) < 1.0 / k)
        drop = drop.to(labels.device)
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
