"""Per-recurrence-step KV cache for the depth-recurrent model.

Semantics are those of the reference's ``HuginnDynamicCache`` (recpre/raven_modeling_minimal.py:148-308): entries are
addressed by ``(step_idx, token position)``; prelude blocks use step indices ``0..P-1``, core iteration j block b uses
``P + R*j + b`` and the coda uses the negative indices ``-1, -2, ...``.  With per-token adaptive depth some positions
lack a given step and a *lookup strategy* decides what to attend to instead (``full``, ``latest-m4``,
``available-m4``, ``always-last-m4``, ``skip``, ``randomized``); ``compress-s{N}`` / ``compress-r{N}`` /
``compress-anchor`` fold step indices onto fewer slots so that the cache is shared across recurrences.

Layout (B200 design): one growing ``[B, capacity, H_kv, D]`` tensor pair per slot -- the layout the attention kernels
read directly, appended in place -- plus a host-side presence bitmap per slot.  The common case (every position
present) returns views without any copy; only the ragged strategies gather.
"""
from __future__ import annotations

import torch


class _Slot:
    __slots__ = ("k", "v", "present")

    def __init__(self):
        self.k = self.v = None
        self.present: list = []

    def ensure(self, like: torch.Tensor, length: int) -> None:
        B, _, H, D = like.shape
        if self.k is None or self.k.shape[1] < length:
            cap = max(64, 1 << (max(length, 1) - 1).bit_length())
            nk = torch.empty(B, cap, H, D, dtype=like.dtype, device=like.device)
            nv = torch.empty_like(nk)
            if self.k is not None:
                n = self.k.shape[1]
                nk[:, :n], nv[:, :n] = self.k, self.v
            self.k, self.v = nk, nv
        if len(self.present) < length:
            self.present.extend([False] * (length - len(self.present)))


class RecurrentKVCache:
    def __init__(self, lookup_strategy: str = "full", core_layers: int = 4, prelude_layers: int = 2):
        self.lookup_strategy = lookup_strategy
        self.R, self.P = core_layers, prelude_layers
        self.slots: dict[int, _Slot] = {}
        self._seen_tokens = 0

    # -- slot index folding ------------------------------------------------------------------------
    def fold(self, step_idx: int) -> int:
        s = self.lookup_strategy
        if "compress-" not in s or step_idx < self.P:
            return step_idx
        P, R = self.P, self.R
        if "compress-s" in s:
            n = int(s.split("compress-")[1][1:])
            return (step_idx - P) % n + P
        if "compress-anchor" in s:
            if step_idx - P < R * 8:
                return step_idx
            base = P + R * 8
            return base + (step_idx - base) % R
        n = int(s.split("compress-")[1][1:])  # compress-r
        return (step_idx - P) // n + P

    # -- main entry ----------------------------------------------------------------------------------
    def update(self, k: torch.Tensor, v: torch.Tensor, step_idx: int, lookup_strategy: str | None = None):
        """Append ``k, v`` of shape [B, S_new, H_kv, D] for the newest S_new positions under ``step_idx`` and return
        the keys/values [B, L, H_kv, D] this step should attend to."""
        step_idx = int(step_idx)
        strategy = self.lookup_strategy if lookup_strategy is None else lookup_strategy
        slot_id = self.fold(step_idx)
        n_new = k.shape[1]
        if slot_id == 0:
            self._seen_tokens += n_new
        seen = self._seen_tokens
        slot = self.slots.setdefault(slot_id, _Slot())
        slot.ensure(k, seen)
        start = seen - n_new
        if "compress-" not in self.lookup_strategy and slot_id >= 0 and any(slot.present[start:seen]):
            raise AssertionError(f"cache entry (step {slot_id}, positions {start}..{seen - 1}) written twice")
        slot.k[:, start:seen] = k
        slot.v[:, start:seen] = v
        for p in range(start, seen):
            slot.present[p] = True
        if all(slot.present[:seen]) or self.lookup_strategy == "full":
            return slot.k[:, :seen], slot.v[:, :seen]
        return self._ragged(slot_id, strategy, seen)

    def _holders(self, pos: int, upto: int | None) -> list:
        return [s for s, sl in self.slots.items()
                if (upto is None or s <= upto) and pos < len(sl.present) and sl.present[pos]]

    def _ragged(self, step_idx: int, strategy: str, seen: int):
        P, R = self.P, self.R
        src = []
        for pos in range(seen):
            here = step_idx in self.slots and self.slots[step_idx].present[pos]
            if strategy.startswith("skip"):
                if here:
                    src.append(step_idx)
                continue
            if step_idx < P:
                src.append(step_idx if here else 0)
                continue
            same = lambda s: s >= P and (s - P) % R == (step_idx - P) % R  # noqa: E731
            if strategy.startswith("latest-m4"):
                src.append(max(s for s in self._holders(pos, step_idx) if same(s)))
            elif strategy.startswith("available-m4"):
                src.append(step_idx if here else max(s for s in self._holders(pos, step_idx) if same(s)))
            elif strategy.startswith("always-last-m4"):
                src.append(max(s for s in self._holders(pos, None) if same(s)))
            elif strategy.startswith("randomized"):
                cands = [s for s in self._holders(pos, step_idx) if same(s)]
                src.append(cands[int(torch.randint(len(cands), (1,)))])
            else:
                raise ValueError(f"Unknown lookup strategy: {strategy}")
        if strategy.startswith("skip"):
            idx = [p for p in range(seen) if self.slots[step_idx].present[p]]
            sl = self.slots[step_idx]
            return sl.k[:, idx], sl.v[:, idx]
        ks = torch.stack([self.slots[s].k[:, p] for p, s in enumerate(src)], dim=1)
        vs = torch.stack([self.slots[s].v[:, p] for p, s in enumerate(src)], dim=1)
        return ks, vs

    # -- bookkeeping -----------------------------------------------------------------------------------
    def reset(self) -> None:
        self.slots.clear()
        self._seen_tokens = 0

    def clear_last_k_entries(self, k: int = 0) -> None:
        """Forget the newest k positions in every slot (speculative / diffusion-style decoding)."""
        assert self._seen_tokens >= k
        self._seen_tokens -= k
        for sl in self.slots.values():
            for p in range(self._seen_tokens, len(sl.present)):
                sl.present[p] = False

    def get_seq_length(self, step_idx: int = 0) -> int:
        return self._seen_tokens

    def get_memory_usage(self) -> float:
        """MiB held by entries that are present (keys and values)."""
        total = 0
        for sl in self.slots.values():
            if sl.k is None:
                continue
            per_pos = sl.k[:, 0].numel() * sl.k.element_size()
            total += per_pos * sum(sl.present)
        return total * 2 / (1024 * 1024)

    def __len__(self) -> int:
        return len(self.slots)


HuginnDynamicCache = RecurrentKVCache


class StaticRecurrentCache:
    """Preallocated cache for the HF-style model (``HuginnStaticCache`` of recpre/raven_modeling_minimal.py:311-437):
    one [batch, max_length, kv heads, head dim] key and value block per step index, written in place, so decoding
    allocates nothing.  Step indices follow the model (prelude 0.., recurrence ``2 + 4 j + b``, coda -1, -2 counted
    from the end of the table); ``compress-s<N>`` / ``compress-r<N>`` fold the recurrence indices into N (resp. every N)
    slots.  Only the ``full`` lookup (every step reads its own entries) and its compressed forms are defined on the
    static layout; the partial-history strategies live in ``RecurrentKVCache``."""

    def __init__(self, max_length: int, max_num_steps: int, num_heads: int, hidden_dim: int, batch_size: int = 1,
                 lookup_strategy: str = "full", device=None, dtype: torch.dtype = torch.float32):
        self.max_length, self.lookup_strategy, self._seen_tokens = max_length, lookup_strategy, 0
        self.stage, self.modulo = 0, False
        if "compress-" in lookup_strategy:
            tag = lookup_strategy.split("compress-")[1]
            self.modulo, self.stage = tag[0] == "s", int(tag[1:].split("-")[0])
            steps = 4 + self.stage if self.modulo else 4 + (max_num_steps - 4 + self.stage - 1) // self.stage
        else:
            steps = max_num_steps
        if not lookup_strategy.startswith(("full", "compress-")):
            raise NotImplementedError(f"lookup strategy {lookup_strategy!r} needs the dynamic cache")
        self.max_num_steps = steps
        shape = (steps, batch_size, max_length, num_heads, hidden_dim)
        self.key_cache = torch.zeros(shape, dtype=dtype, device=device)
        self.value_cache = torch.zeros(shape, dtype=dtype, device=device)
        self.valid_mask = torch.zeros(steps, max_length, dtype=torch.bool, device=device)

    def fold(self, step_idx: int) -> int:
        step_idx = int(step_idx)
        if self.stage and step_idx > 1:
            return (step_idx - 2) % self.stage + 2 if self.modulo else (step_idx - 2) // self.stage + 2
        return step_idx

    def update(self, k: torch.Tensor, v: torch.Tensor, step_idx: int, lookup_strategy: str | None = None):
        """k, v: [B, S_new, Hkv, D] of the newest positions; returns the step's keys and values of all positions."""
        n = k.shape[1]
        if int(step_idx) == 0:
            self._seen_tokens += n
        assert self._seen_tokens <= self.max_length, "static cache is full"
        slot = self.fold(step_idx)
        lo = self._seen_tokens - n
        B = k.shape[0]
        self.key_cache[slot, :B, lo:lo + n].copy_(k)
        self.value_cache[slot, :B, lo:lo + n].copy_(v)
        self.valid_mask[slot, lo:lo + n] = True
        return self.key_cache[slot, :B, :self._seen_tokens], self.value_cache[slot, :B, :self._seen_tokens]

    def reset(self) -> None:
        self._seen_tokens = 0
        self.key_cache.zero_()
        self.value_cache.zero_()
        self.valid_mask.zero_()

    def clear_last_k_entries(self, k: int = 0) -> None:
        assert self._seen_tokens >= k
        self._seen_tokens -= k
        self.valid_mask[:, self._seen_tokens:] = False

    def get_seq_length(self, step_idx: int = 0) -> int:
        return self._seen_tokens

    def get_memory_usage(self) -> float:
        return (self.key_cache.nelement() + self.value_cache.nelement()) * self.key_cache.element_size() / (1024 * 1024)


HuginnStaticCache = StaticRecurrentCache
