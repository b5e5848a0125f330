"""Weight-initialisation strategies selected by name.

Behavioural contract (recpre/init.py:27-171,312-479): a strategy is a table of standard deviations keyed by layer role
(``embedding``, ``in_proj``, ``out_proj``, ``head``, ``q`` / ``k`` / ``v``, ``out_attn``, ``mlp``, ``std`` as the
fallback) plus multipliers (``embed_scale``, ``logit_scale``, ``residual``, ``skip``).  Normals are truncated at
+-3 sigma unless ``truncate_normals`` is off; ``orthogonal`` swaps the normal for a (truncated-normal seeded) orthogonal
matrix of the same entry scale; the ``bernstein`` strategy uses orthogonal matrices at their natural scale
sqrt(fan_out / fan_in).  Fused tensors are initialised per part: ``Wqkv`` rows are ``[Q; K; V]`` and ``fc`` rows of a
gated MLP are ``[gate; up]`` (both halves with the ``w1`` deviation, as in the reference).

Two lookups exist, and they differ in the reference (its ``get_std`` / ``get_scales`` / ``logit_scale`` /
``embedding_scale`` hand their arguments to the table positionally, one place off): weights (``fn`` /
``init_weight_``) see the real layer index, depth and head size, with widths divided by the muP factor; the scalar
queries see the full widths, the QUERIED LAYER INDEX AS HEAD SIZE, the model depth as layer index and a depth of 16.
Models built here must match models built there, so both lookups are kept as they are (``takase`` and ``scaled`` are
not affected: their ``embedding`` / ``std`` entries depend on neither).
"""
from __future__ import annotations

import math
from math import sqrt
from typing import Callable, Optional

import torch

STRATEGIES = ("mitchell", "normal", "llama", "llama-by-dim", "llama-by-dim-ls", "kaiming", "bert", "megatron",
              "megatron2", "small", "scaled", "scaled-stuck", "takase", "takase-scaled", "wang", "deepnorm-straight",
              "deepnorm-subln", "noci-anagnostidis", "shaped", "deep-scale-simple", "deep-scale-full",
              "scaled-and-logit-scale", "bernstein", "illiterate", "scaled-large-embed", "zero-out")


def _xavier_std(gain: float, fan_a: int, fan_b: int) -> float:
    return gain * sqrt(2.0 / float(fan_a + fan_b))


def _deepscale_value_std(dim: int, num_layers: int, layer_idx: int) -> float:
    """Value / attention-output deviation of DeepScaleLM for one layer: the input correlation r is propagated through
    the attention and MLP blocks of a lambda^2 = 1 - 2/N, beta^2 = 2/N residual stack (no dropout), starting from the
    Zipf-law estimate r0 = 0.221 (recpre/init.py:174-204)."""
    lam2, beta2 = 1 - 2 / num_layers, 2 / num_layers
    r, var = 0.221, 1.0
    per_layer = []
    for _ in range(num_layers):
        per_layer.append(sqrt(sqrt(1.0 / r) / dim))
        r = (lam2 * r * var + beta2 * 1.0) / (lam2 * var + beta2)            # attention block: output correlation 1
        var = lam2 * var + beta2
        r_mlp = r + (sqrt(1 - r * r) - r * math.acos(r)) / math.pi          # ReLU block
        r = (lam2 * r * var + beta2 * r_mlp) / (lam2 * var + beta2)
        var = lam2 * var + beta2
    return per_layer[layer_idx]


def strategy_table(strategy: str, dim: int, dim2: int, head_dim: int, layer_idx: int = 0, num_layers: int = 16) -> dict:
    """Deviations and multipliers of one strategy for one layer."""
    L = int(num_layers)
    li = layer_idx % L
    base = sqrt(2 / (5 * dim))
    inv = 1 / sqrt(dim)
    if strategy == "mitchell":
        return {"embedding": inv, "head": inv, "in_proj": inv, "out_proj": inv / sqrt(2 * (li + 1))}
    if strategy == "normal":
        return {"std": inv}
    if strategy == "llama":
        return {"embedding": 1.0, "in_proj": 0.02, "out_proj": 0.02 / sqrt(2 * (li + 1)), "head": inv}
    if strategy == "llama-by-dim":
        return {"embedding": 1.0, "in_proj": inv, "out_proj": inv / sqrt(2 * (li + 1)), "head": inv}
    if strategy == "llama-by-dim-ls":
        return {"embedding": 1.0, "in_proj": inv, "out_proj": inv / sqrt(2 * (li + 1)), "head": 1.0, "logit_scale": inv}
    if strategy == "kaiming":
        return {"std": sqrt(2.0 / dim)}
    if strategy == "bert":
        return {"std": 0.02}
    if strategy == "megatron":
        return {"std": 0.02, "out_proj": 0.02 / sqrt(dim), "embedding": 0.02, "head": inv}
    if strategy == "megatron2":
        return {"std": sqrt(1 / (3 * dim))}
    if strategy == "small":
        return {"std": base}
    if strategy == "scaled":
        return {"std": base, "out_proj": base / sqrt(2 * L)}
    if strategy == "scaled-stuck":
        return {"std": base, "out_proj": base / sqrt(2 * 16)}
    if strategy == "takase":
        return {"std": base, "out_proj": base / sqrt(2 * L), "embedding": base, "embed_scale": sqrt(dim)}
    if strategy == "takase-scaled":
        return {"std": base, "out_proj": base / sqrt(2 * L), "embedding": base, "embed_scale": sqrt(dim),
                "logit_scale": sqrt(2 / 5) / sqrt(dim)}
    if strategy == "wang":
        return {"std": 2 / L / sqrt(dim)}
    if strategy == "deepnorm-straight":
        gain = pow(8 * L, -0.25)
        return {"embedding": 0.02, "gain": gain, "skip": pow(2 * L, 0.25), "mlp": _xavier_std(gain, dim, dim2),
                "out_proj": _xavier_std(gain, dim, dim2), "v": _xavier_std(gain, dim, dim),
                "out_attn": _xavier_std(gain, dim, dim), "q": _xavier_std(1.0, dim, head_dim),
                "k": _xavier_std(1.0, dim, head_dim), "head": inv}
    if strategy == "deepnorm-subln":
        gain = sqrt(math.log(2 * L))
        return {"embedding": 0.02, "gain": gain, "skip": pow(2 * L, 0.25), "mlp": _xavier_std(gain, dim, dim2),
                "v": _xavier_std(gain, dim, dim), "out_attn": _xavier_std(gain, dim, dim),
                "q": _xavier_std(1.0, dim, head_dim), "k": _xavier_std(1.0, dim, head_dim), "head": inv}
    if strategy == "noci-anagnostidis":
        return {"residual": 1 / sqrt(L), "mlp": _xavier_std(1.0, dim, dim2), "v": _xavier_std(1.0, dim, dim),
                "out_attn": _xavier_std(1.0, dim, dim), "q": _xavier_std(1.0, dim, head_dim),
                "k": _xavier_std(1.0, dim, head_dim), "std": 1.0, "logit_scale": inv}
    if strategy == "shaped":                   # goes with identity-shaped activation functions
        return {"residual": 0.2, "skip": sqrt(1 - 0.2 ** 2), "in_proj": inv, "out_proj": inv, "std": 1.0, "q": inv,
                "k": inv, "logit_scale": inv}
    if strategy in ("deep-scale-simple", "deep-scale-full"):
        t = {"residual": sqrt(2 / L), "skip": sqrt(1 - 2 / L), "std": sqrt(1 / dim * sqrt(1 / 2)), "q": inv, "k": inv,
             "embedding": sqrt(1 / 3), "head": 1.0, "logit_scale": inv}
        if strategy.endswith("full"):
            t["v"] = t["out_attn"] = _deepscale_value_std(dim, L, li)
        return t
    if strategy == "scaled-and-logit-scale":
        return {"std": base, "out_proj": base / sqrt(2 * L), "embedding": 1.0, "head": inv, "logit_scale": inv}
    if strategy == "bernstein":                # orthogonal matrices at their natural scale (see Init)
        return {"std": 1.0}
    if strategy == "illiterate":
        return {"embedding": 1.0, "std": inv, "out_proj": 0.0, "head": 0.0}
    if strategy == "scaled-large-embed":
        return {"embedding": 1.0, "std": inv, "out_proj": inv / sqrt(2 * L)}
    if strategy == "zero-out":                 # not in the reference: `small` with zero output projections
        return {"std": base, "out_proj": 0.0}
    raise ValueError(f"unknown init strategy {strategy!r}")


# ------------------------------------------------------------------------------------------ tensor fillers
def trunc_normal_(t: torch.Tensor, std: float, generator=None) -> torch.Tensor:
    if std == 0.0:
        return t.zero_()
    return torch.nn.init.trunc_normal_(t, mean=0.0, std=std, a=-3 * std, b=3 * std, generator=generator)


def plain_normal_(t: torch.Tensor, std: float) -> torch.Tensor:
    return torch.nn.init.normal_(t, mean=0.0, std=std)


@torch.no_grad()
def _orthogonal_from_trunc_normal_(t: torch.Tensor, gain: float) -> torch.Tensor:
    """Orthonormal rows or columns from the QR factorisation of a truncated-normal matrix (signs fixed by the diagonal
    of R so that the factor is uniformly distributed), times ``gain`` (recpre/init.py:207-235)."""
    rows = t.size(0)
    cols = t.numel() // rows
    flat = t.new_empty(rows, cols)
    torch.nn.init.trunc_normal_(flat, mean=0.0, std=1.0)
    if rows < cols:
        flat = flat.t()
    q, r = torch.linalg.qr(flat)
    q = q * torch.diag(r, 0).sign()
    if rows < cols:
        q = q.t()
    t.view(rows, cols).copy_(q)
    return t.mul_(gain)


def trunc_orthogonal_(t: torch.Tensor, std: float) -> torch.Tensor:
    """Orthogonal matrix scaled so that its entries have deviation about ``std``."""
    if t.ndim < 2:
        return trunc_normal_(t, std)
    return _orthogonal_from_trunc_normal_(t, std * sqrt(max(t.shape[0], t.numel() // t.shape[0])))


def orthogonal_(t: torch.Tensor, std: float) -> torch.Tensor:
    return torch.nn.init.orthogonal_(t, gain=std * sqrt(max(t.shape[0], t.numel() // t.shape[0])))


def natural_scale_orthogonal_(t: torch.Tensor, std: float = 1.0) -> torch.Tensor:
    fan_out = t.shape[0]
    return _orthogonal_from_trunc_normal_(t, std * sqrt(fan_out / (t.numel() // fan_out)))


_DIVIDED_BY_MUP = ("out_attn", "w1", "w2", "w3", "q", "k", "v", "mlp", "in_proj", "out_proj")


class Init:
    """Dispatches the initialisers of one model.  Argument names follow the reference (``init_strategy``,
    ``mup_model_scaling_factor``, ``skip_reinitializing``); ``strategy`` / ``mup`` / ``skip`` are shorter aliases."""

    def __init__(self, init_strategy: str = "mitchell", dim: int = 1024, dim2: int = 4096, head_dim: int = 64,
                 num_layers: int = 32, mup_model_scaling_factor: int = 1, truncate_normals: bool = True,
                 orthogonal: bool = False, verbose: bool = False, skip_reinitializing: bool = False, *,
                 strategy: Optional[str] = None, mup: Optional[int] = None, skip: Optional[bool] = None):
        self.strategy = self.init_strategy = strategy if strategy is not None else init_strategy
        self.dim, self.dim2, self.head_dim, self.num_layers = dim, dim2, head_dim, num_layers
        self.mup = self.mup_model_scaling_factor = mup if mup is not None else mup_model_scaling_factor
        self.skip = self.skip_reinitializing = skip if skip is not None else skip_reinitializing
        self.verbose = verbose
        if "bernstein" in self.strategy:
            self.normal_: Callable = natural_scale_orthogonal_
        elif orthogonal:
            self.normal_ = trunc_orthogonal_ if truncate_normals else orthogonal_
        else:
            self.normal_ = trunc_normal_ if truncate_normals else plain_normal_
        strategy_table(self.strategy, dim, dim2, head_dim, 0, num_layers)  # validates the name early

    # --- scalar queries (the reference's one-place-off lookup, see the module docstring) -------------------------
    def _query_table(self, layer_idx: int) -> dict:
        return strategy_table(self.strategy, self.dim, self.dim2, layer_idx, self.num_layers, 16)

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
            raise ValueError(f"layer {role!r} asks for the undefined init key 'std'; rename the layer to match the table")
        return table["std"]

    def get_std(self, role: str, layer_idx: int = -1) -> float:
        return float(self._resolve(self._query_table(layer_idx), role))

    def get_scales(self, layer_idx: int = -1) -> tuple[float, float]:
        t = self._query_table(layer_idx)
        return float(t.get("residual", 1.0)), float(t.get("skip", 1.0))

    @property
    def embedding_scale(self) -> float:
        return float(self._query_table(0).get("embed_scale", 1.0))

    @property
    def logit_scale(self) -> float:
        return float(self._query_table(0).get("logit_scale", 1.0)) / self.mup

    # --- tensor initialisers ----------------------------------------------------------------------------------------
    def fn(self, name_of_layer: str, layer_idx: int = 0) -> Callable:
        """The initialiser of one layer as a callable on its weight (what ``Linear(init_method=...)`` stores)."""
        return lambda tensor: self.init_weight_(tensor, name_of_layer, layer_idx)

    def apply(self, module, name_of_layer: Optional[str] = None, layer_idx: int = 0) -> None:
        """Initialise an already constructed module: its weight by role, its bias with zeros."""
        if name_of_layer is not None and hasattr(module, "weight"):
            self.init_weight_(module.weight, name_of_layer, layer_idx)
        if getattr(module, "bias", None) is not None:
            torch.nn.init.zeros_(module.bias)

    def init_weight_(self, tensor: torch.Tensor, role: str, layer_idx: int = 0) -> None:
        """Initialise ``tensor`` in place for the given role.  Roles: ``embedding``, ``head``, ``qkv`` (fused [Q;K;V];
        ``qkv-diagonal``: Q and K scaled identities), ``glu`` (fused [gate;up]), ``in_proj``, ``out_proj``,
        ``out_attn``, ``q`` / ``k`` / ``v``, ``w1`` / ``w2`` / ``w3``, ``mlp``, ``normalization``."""
        if self.skip:
            return
        mu = self.mup
        table = strategy_table(self.strategy, self.dim // mu, self.dim2 // mu, self.head_dim, layer_idx, self.num_layers)
        with torch.no_grad():
            if "normalization" in role:
                tensor.fill_(1.0)
            elif "qkv" in role:
                qk = next(table[k] for k in ("q", "in_proj", "std") if k in table) / mu
                v = next(table[k] for k in ("v", "in_proj", "std") if k in table) / mu
                kv_rows = (tensor.shape[0] - self.dim) // (2 * self.head_dim) * self.head_dim
                q_part, k_part, v_part = tensor.split([self.dim, kv_rows, kv_rows], dim=0)
                if "diagonal" in role:
                    assert kv_rows == self.dim, "diagonal q/k need as many key heads as query heads"
                    eye = torch.eye(self.dim, dtype=tensor.dtype, device=tensor.device) * float(qk)
                    q_part.copy_(eye)
                    k_part.copy_(eye)
                else:
                    self.normal_(q_part, std=float(qk))
                    self.normal_(k_part, std=float(qk))
                self.normal_(v_part, std=float(v))
            elif "glu" in role:
                w1 = next(table[k] for k in ("w1", "mlp", "in_proj", "std") if k in table) / mu
                for part in tensor.chunk(2, dim=0):  # both halves use the w1 deviation (recpre/init.py:399)
                    self.normal_(part, std=float(w1))
            else:
                std = self._resolve(table, role)
                named_or_proj = role in table or ("out_proj" in table and role in ("out_attn", "w2", "w3")) or \
                    ("in_proj" in table and role in ("q", "k", "v", "w1")) or \
                    ("mlp" in table and role in ("w1", "w2", "w3", "mlp"))
                if named_or_proj and role in _DIVIDED_BY_MUP:   # the `std` fallback and embedding / head stay undivided
                    std = std / mu
                self.normal_(tensor, std=float(std))

    def __repr__(self) -> str:
        return f"{self.strategy} Initializer {self.dim}x{self.dim2}x{self.head_dim}-{self.num_layers}"
