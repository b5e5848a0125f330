"""Weight-initialisation strategies selected by name.

Behavioural contract (recpre/init.py:27-171,312-479): a strategy is a table of standard
deviations keyed by layer role (``embedding``, ``in_proj``, ``out_proj``, ``head``, ``std``
fallback, plus ``embed_scale`` / ``logit_scale`` multipliers).  All normals are truncated
at +-3 sigma unless an orthogonal variant is requested.  Fused tensors are initialised per
part: ``Wqkv`` rows are ``[Q; K; V]`` and ``fc`` rows of a gated MLP are ``[gate; up]``.

The reference evaluates depth-dependent entries with a fallback depth of 16 when std values
are queried through ``get_std`` (recpre/init.py:449-475 passes arguments positionally);
``takase``/``scaled`` std for ``embedding`` does not depend on depth so the state-init sigma
is unaffected.  ``fn`` (used for weights) does use the real depth.
"""
from __future__ import annotations

import math
from math import sqrt
from typing import Callable

import torch


def _xavier_std(gain: float, fan_in: int, fan_out: int) -> float:
    return gain * sqrt(2.0 / (fan_in + fan_out))


def strategy_table(strategy: str, dim: int, dim2: int, head_dim: int, layer_idx: int, num_layers: int) -> dict:
    L = max(int(num_layers), 1)
    li = layer_idx % L
    base = sqrt(2 / (5 * dim))
    if strategy == "mitchell":
        s = 1 / sqrt(dim)
        return {"embedding": s, "head": s, "in_proj": s, "out_proj": s / sqrt(2 * (li + 1))}
    if strategy == "normal":
        return {"std": 1 / sqrt(dim)}
    if strategy == "llama":
        return {"embedding": 1.0, "in_proj": 0.02, "out_proj": 0.02 / sqrt(2 * (li + 1)), "head": 1 / sqrt(dim)}
    if strategy in ("llama-by-dim", "llama-by-dim-ls"):
        t = {"embedding": 1.0, "in_proj": 1 / sqrt(dim), "out_proj": 1 / sqrt(dim) / sqrt(2 * (li + 1)),
             "head": 1 / sqrt(dim)}
        if strategy.endswith("-ls"):
            t.update(head=1.0, logit_scale=1 / sqrt(dim))
        return t
    if strategy == "kaiming":
        return {"std": sqrt(2.0 / dim)}
    if strategy == "bert":
        return {"std": 0.02}
    if strategy == "megatron":
        return {"std": 0.02, "out_proj": 0.02 / sqrt(dim), "embedding": 0.02, "head": 1 / sqrt(dim)}
    if strategy == "megatron2":
        return {"std": sqrt(1 / (3 * dim))}
    if strategy == "small":
        return {"std": base}
    if strategy == "scaled":
        return {"std": base, "out_proj": base / sqrt(2 * L)}
    if strategy == "scaled-stuck":
        return {"std": base, "out_proj": base / sqrt(2 * 16)}
    if strategy in ("takase", "takase-scaled"):
        t = {"std": base, "out_proj": base / sqrt(2 * L), "embedding": base, "embed_scale": sqrt(dim)}
        if strategy == "takase-scaled":
            t["logit_scale"] = sqrt(2 / 5) / sqrt(dim)
        return t
    if strategy == "wang":
        return {"std": 2 / L / sqrt(dim)}
    if strategy in ("deepnorm-straight", "deepnorm-subln"):
        gain = pow(8 * L, -0.25) if strategy.endswith("straight") else sqrt(math.log(2 * L))
        t = {"embedding": 0.02, "gain": gain, "skip": pow(2 * L, 0.25), "mlp": _xavier_std(gain, dim, dim2),
             "v": _xavier_std(gain, dim, dim), "out_attn": _xavier_std(gain, dim, dim),
             "q": _xavier_std(1.0, dim, head_dim), "k": _xavier_std(1.0, dim, head_dim), "head": 1 / sqrt(dim)}
        if strategy.endswith("straight"):
            t["out_proj"] = _xavier_std(gain, dim, dim2)
        return t
    if strategy == "noci-anagnostidis":
        return {"residual": 1 / sqrt(L), "std": 1 / sqrt(dim)}
    if strategy == "zero-out":
        return {"std": base, "out_proj": 0.0}
    raise ValueError(f"unknown init strategy {strategy!r}")


def trunc_normal_(t: torch.Tensor, std: float, generator=None) -> torch.Tensor:
    if std == 0.0:
        return t.zero_()
    return torch.nn.init.trunc_normal_(t, mean=0.0, std=std, a=-3 * std, b=3 * std, generator=generator)


def trunc_orthogonal_(t: torch.Tensor, std: float) -> torch.Tensor:
    """Orthogonal matrix rescaled so that its entries have standard deviation ``std``."""
    if t.ndim < 2 or std == 0.0:
        return trunc_normal_(t, std)
    with torch.no_grad():
        rows, cols = t.shape[0], t[0].numel()
        flat = torch.empty(rows, cols, dtype=torch.float32)
        torch.nn.init.orthogonal_(flat)
        flat.mul_(std * sqrt(max(rows, cols)))
        t.copy_(flat.view_as(t).clamp_(-3 * std, 3 * std))
    return t


class Init:
    def __init__(self, strategy: str = "scaled", dim: int = 1024, dim2: int = 4096, head_dim: int = 64,
                 num_layers: int = 32, mup: int = 1, orthogonal: bool = False, skip: bool = False):
        self.strategy, self.dim, self.dim2, self.head_dim = strategy, dim, dim2, head_dim
        self.num_layers, self.mup, self.skip = num_layers, mup, skip
        self.normal_: Callable = trunc_orthogonal_ if orthogonal else trunc_normal_
        strategy_table(strategy, dim, dim2, head_dim, 0, num_layers)  # validates the name early

    # --- std lookups ------------------------------------------------------------
    def _table(self, layer_idx: int = 0, depth: int | None = None) -> dict:
        mu = self.mup
        return strategy_table(self.strategy, self.dim // mu, self.dim2 // mu, self.head_dim, layer_idx,
                              self.num_layers if depth is None else depth)

    @staticmethod
    def _resolve(table: dict, role: str) -> float:
        if role in table:
            return table[role]
        if "out_proj" in table and role in ("out_attn", "w2", "w3"):
            return table["out_proj"]
        if "in_proj" in table and role in ("q", "k", "v", "w1"):
            return table["in_proj"]
        if "mlp" in table and role in ("w1", "w2", "w3", "mlp"):
            return table["mlp"]
        if "std" not in table:
            raise ValueError(f"init strategy {role!r} undefined")
        return table["std"]

    def get_std(self, role: str, layer_idx: int = -1) -> float:
        # depth fallback of 16 replicates the reference's positional-argument behaviour
        return float(self._resolve(strategy_table(self.strategy, self.dim, self.dim2, self.head_dim, 0, 16), role))

    @property
    def embedding_scale(self) -> float:
        return float(self._table().get("embed_scale", 1.0))

    @property
    def logit_scale(self) -> float:
        return float(self._table().get("logit_scale", 1.0)) / self.mup

    def get_scales(self, layer_idx: int = -1) -> tuple[float, float]:
        t = self._table()
        return float(t.get("residual", 1.0)), float(t.get("skip", 1.0))

    # --- tensor initialisers ----------------------------------------------------
    def init_weight_(self, tensor: torch.Tensor, role: str, layer_idx: int = 0) -> None:
        """Initialise ``tensor`` in place for the given role.  Roles: ``embedding``, ``head``,
        ``qkv`` (fused [Q;K;V]), ``glu`` (fused [gate;up]), ``in_proj``, ``out_proj``,
        ``out_attn``, ``w1``/``w2``/``w3``, ``normalization``."""
        if self.skip:
            return
        table = self._table(layer_idx)
        mu = self.mup
        with torch.no_grad():
            if role == "normalization":
                tensor.fill_(1.0)
            elif role == "qkv":
                qk = next(table[k] for k in ("q", "in_proj", "std") if k in table) / mu
                v = next(table[k] for k in ("v", "in_proj", "std") if k in table) / mu
                kv_rows = (tensor.shape[0] - self.dim) // 2
                parts = tensor.split([self.dim, kv_rows, kv_rows], dim=0)
                for part, std in zip(parts, (qk, qk, v)):
                    self.normal_(part, std=float(std))
            elif role == "glu":
                w1 = next(table[k] for k in ("w1", "mlp", "in_proj", "std") if k in table) / mu
                for part in tensor.chunk(2, dim=0):  # both halves use the w1 std (recpre/init.py:399)
                    self.normal_(part, std=float(w1))
            else:
                std = self._resolve(table, role)
                if role not in ("embedding", "head"):
                    std = std / mu
                self.normal_(tensor, std=float(std))

    def __repr__(self) -> str:
        return f"Init({self.strategy}, {self.dim}x{self.dim2}x{self.head_dim}, depth {self.num_layers})"
