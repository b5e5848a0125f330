"""Model configuration objects.

Field names follow the reference's model config (recpre/config_dynamic.py:36-92,
354-419) so that registry dicts, ``model_overwrite`` entries from launch YAMLs and the
``model_config`` dict stored in checkpoints stay interchangeable.  Construction of the
actual modules lives in ``models``; this module only validates and derives shapes.
"""
from __future__ import annotations

import copy
import dataclasses
import math
from dataclasses import dataclass, field
from typing import Any, Optional

from . import registry


@dataclass
class RoPESettings:
    """recpre/config_dynamic.py:29-33."""

    use_rope: bool = True
    rope_condense_ratio: int = 1
    rope_base: int = 50_000


def _round_up(n: int, k: int) -> int:
    return n if n % k == 0 else n + k - (n % k)


@dataclass
class ModelConfig:
    name: str = ""
    hf_config: dict = field(default_factory=dict)
    architecture_class_name: str = "GPT"  # GPT | RecurrentGPT
    # core
    block_size: int = 4096
    n_embd: int = 4096
    intermediate_size: Optional[int] = None
    num_attention_heads: int = 32
    num_key_value_heads: Optional[int] = None
    # embeddings
    vocab_size: int = 50254
    padding_multiple: int = 512
    padded_vocab_size: Optional[int] = None
    rope_settings: RoPESettings = field(default_factory=RoPESettings)
    use_abacus: bool = False
    abacus_ids: list = field(default_factory=lambda: list(range(10)))
    randomize_positions_from: Optional[int] = None
    scale_embeddings: bool = False
    # blocks
    block_class_name: str = "TransformerPreNormBlock"
    norm_class_name: str = "LayerNorm"
    attn_impl: str = "sdpa"
    norm_eps: float = 1e-5
    mlp_class_name: str = "BaseMLP"
    nonlin_name: str = "GELU"
    bias: bool = False
    qk_bias: bool = False
    lm_head_bias: bool = False
    init_strategy: str = "scaled"
    init_orthogonal: bool = False
    skip_initialization: bool = False
    mup_model_scaling_factor: int = 1
    use_fused_head: str = "pytorch"  # hhe | cce | full-triton | pytorch | b200 (fused linear+CE kernel)
    loss_shape: str = "none"
    mod_capacity_factor: float = 0.125
    debias_attention: bool = False
    center_attention: bool = False
    clip_qkv: Optional[float] = None
    qk_norm: bool = False
    activation_checkpoint_impl: Optional[str] = None   # default: per-iteration (recurrent) / per-block (GPT)
    simple_ops: bool = False
    strategy: str = "single"
    # GPT only
    n_layer: int = 16
    # recurrent only (recpre/config_dynamic.py:392-419)
    injection_type: str = "add"  # none | add | gate | linear | ffn | modulated
    embed_step: bool = False
    randomize_embed_step: bool = False
    normalize_rec: str = ""
    intermediate_noise_injection: float = 0.0
    geom_noise_injection: str = "geom"
    n_layers_in_recurrent_block: int = 4
    n_layers_in_prelude: int = 1
    n_layers_in_coda: int = 1
    state_init: str = "like-init"  # normal | embed | like-init | zero | unit
    sampling_scheme: str = "poisson-unbounded"
    mean_recurrence: int = 32
    mean_backprop_depth: int = 8
    lockstep_n: bool = False
    lockstep_k: bool = False
    mcleish_throttle: bool = False
    elbayad_weighing: bool = False
    elbayad_exponent: float = 1.0
    seers: int = 0
    tie_embeddings: bool = False
    # knob added here: multiplies the state-init standard deviation.  The default
    # reproduces the reference's sigma = sqrt(2/(5E)) * sqrt(E) = sqrt(0.4).
    state_init_scale: float = 1.0

    def __post_init__(self):
        if isinstance(self.rope_settings, dict):
            self.rope_settings = RoPESettings(**self.rope_settings)
        if not self.name:
            self.name = self.hf_config.get("name", self.name)
        if self.padded_vocab_size is None:
            self.padded_vocab_size = _round_up(self.vocab_size, self.padding_multiple)
        else:
            self.vocab_size = min(self.vocab_size, self.padded_vocab_size)
        if self.activation_checkpoint_impl is None:    # the two config classes of the reference differ here
            self.activation_checkpoint_impl = "per-iteration" if self.architecture_class_name == "RecurrentGPT" \
                else "per-block"
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        if self.n_embd % self.num_attention_heads:
            raise ValueError("n_embd must be divisible by num_attention_heads")
        self.head_size = self.n_embd // self.num_attention_heads
        if self.intermediate_size is None:
            self.intermediate_size = 4 * self.n_embd
        mu = self.mup_model_scaling_factor
        self.n_embd *= mu
        self.intermediate_size *= mu
        self.num_key_value_heads *= mu
        self.n_head = self.num_attention_heads * mu
        self.n_query_groups = self.num_key_value_heads
        if self.is_recurrent:
            # effective depth used by depth-aware init strategies
            self.effective_expected_depth = (
                self.n_layers_in_prelude
                + self.n_layers_in_coda
                + self.n_layers_in_recurrent_block * self.mean_recurrence
            )
            self.n_layer = self.n_layers_in_recurrent_block * self.mean_backprop_depth
            depth_for_init = self.effective_expected_depth
        else:
            self.effective_expected_depth = self.n_layer
            depth_for_init = self.n_layer
        from .models.init import Init

        self.init = Init(
            self.init_strategy,
            self.n_embd,
            self.intermediate_size,
            self.head_size,
            depth_for_init,
            mu,
            orthogonal=self.init_orthogonal,
            skip=self.skip_initialization,
        )

    # ------------------------------------------------------------------
    @property
    def is_recurrent(self) -> bool:
        return self.architecture_class_name == "RecurrentGPT"

    @property
    def rope_n_elem(self) -> int:
        return self.head_size

    @classmethod
    def from_name(cls, name: str, **overrides: Any) -> "ModelConfig":
        """Registry lookup plus overrides; ``rope_settings.<key>`` overrides are dotted
        (recpre/config_dynamic.py:128-155)."""
        d = registry.lookup(name)
        rope: dict = {}
        for k, v in overrides.items():
            if k.startswith("rope_settings."):
                rope[k.split(".", 1)[1]] = v
            else:
                d[k] = v
        if rope:
            base = d.get("rope_settings", {})
            if isinstance(base, RoPESettings):
                base = dataclasses.asdict(base)
            d["rope_settings"] = RoPESettings(**{**base, **rope})
        return cls.from_dict(d)

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        known = {f.name for f in dataclasses.fields(cls)}
        unknown = set(d) - known
        if unknown:
            raise ValueError(f"unknown model config keys: {sorted(unknown)}")
        if d.get("architecture_class_name", "GPT") not in ("GPT", "RecurrentGPT"):
            raise ValueError(f"Invalid architecture {d['architecture_class_name']} provided.")
        return cls(**d)

    def to_dict(self) -> dict:
        out = {}
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            if dataclasses.is_dataclass(v):
                v = dataclasses.asdict(v)
            out[f.name] = v
        # undo the mup scaling so that from_dict(to_dict()) round-trips
        mu = self.mup_model_scaling_factor
        out["n_embd"] = self.n_embd // mu
        out["intermediate_size"] = self.intermediate_size // mu
        out["num_key_value_heads"] = self.num_key_value_heads // mu
        return out

    @classmethod
    def from_json(cls, path, **overrides: Any) -> "ModelConfig":
        """A config stored as JSON (``lit_config.json`` / ``model_config.json``), keyword overrides applied on top."""
        import json

        with open(path, encoding="utf-8") as fp:
            d = json.load(fp)
        d.update(overrides)
        d.pop("init", None)
        return cls.from_dict(d)

    @classmethod
    def from_checkpoint(cls, path, **overrides: Any) -> "ModelConfig":
        """``<path>/lit_config.json`` if it exists, else the registry entry named like the directory
        (recpre/config_dynamic.py:168-174)."""
        from pathlib import Path

        path = Path(path)
        if (path / "lit_config.json").is_file():
            return cls.from_json(path / "lit_config.json", **overrides)
        if path.name in registry.name_to_config:
            return cls.from_name(path.name, **overrides)
        raise FileNotFoundError(f"For {str(path)!r} neither 'lit_config.json' nor matching config exists.")

    # class lookups by the names stored in the config (recpre/config_dynamic.py:176-251) -------------------------------
    @property
    def MLP(self):
        from .models.blocks import MLP_CLASSES

        return MLP_CLASSES[self.mlp_class_name]

    @property
    def Block(self):
        from .models.blocks import BLOCK_CLASSES

        return BLOCK_CLASSES[self.block_class_name]

    @property
    def Linear(self):
        from .models.blocks import Linear

        return Linear

    @property
    def Nonlin(self):
        import torch.nn as nn

        from .models.blocks import Relu2

        if hasattr(nn, self.nonlin_name):
            return getattr(nn, self.nonlin_name)
        if self.nonlin_name == "ReLU2":
            return Relu2
        raise ValueError(f"Could not identify nonlinearity {self.nonlin_name}")

    @property
    def Norm(self):
        """``cfg.Norm(size, eps=...)`` builds the configured norm."""
        from .models.blocks import make_norm

        def build(size: int, eps: Optional[float] = None, **_):
            if eps is None or eps == self.norm_eps:
                return make_norm(self, size)
            other = copy.copy(self)                   # a shallow copy: the constructor would apply the muP widths again
            other.norm_eps = eps
            return make_norm(other, size)

        return build

    @property
    def attn_nonlin_fn(self):
        """Factory of the attention computation ``f(q, k, v, mask)`` on [B, S, H, D] tensors for the configured provider
        options (centering, causal-mean debiasing, soft cap); the models' attention modules apply the same options
        themselves."""
        from .models.blocks import _center_debias, _dense_attention

        softcap = 20.0 if self.attn_impl == "flex-attention-soft-cap" else 0.0
        center, debias = bool(self.center_attention), bool(self.debias_attention)

        def factory():
            def attend(q, k, v, mask=None):
                if self.attn_impl == "debug-skip":
                    return v
                y = _dense_attention(q, k, v, softcap)
                return _center_debias(y, v, q.shape[2], center, debias) if (center or debias) else y

            return attend

        return factory

    @property
    def checkpoint(self):
        """The activation-checkpoint callable of ``activation_checkpoint_impl`` (plain, ``sac``, ``sac-attn``,
        ``sac%N``)."""
        from .ops.sac import checkpoint_fn

        return checkpoint_fn(self.activation_checkpoint_impl)

    def __getstate__(self):
        state = dict(self.__dict__)
        state.pop("init", None)                        # rebuilt from the fields
        return state

    def __setstate__(self, state):
        self.__dict__.update(state)
        from .models.init import Init

        depth = self.effective_expected_depth if self.is_recurrent else self.n_layer
        self.init = Init(self.init_strategy, self.n_embd, self.intermediate_size, self.head_size, depth,
                         self.mup_model_scaling_factor, orthogonal=self.init_orthogonal, skip=self.skip_initialization)

    def construct_model(self, **kwargs):
        """recpre/config_dynamic.py:441-444: ``cfg.construct_model(objective=..., gradient_checkpointing=...)``."""
        from .models import build_model

        return build_model(self, **kwargs)

    # parameter / FLOP bookkeeping -------------------------------------------------
    def param_count(self) -> int:
        E, I, V = self.n_embd, self.intermediate_size, self.padded_vocab_size
        hd = self.head_size
        kv = self.num_key_value_heads * hd
        gated = self.mlp_class_name.startswith("Gated")
        per_block = (E + 2 * kv) * E + E * E + (2 * I if gated else I) * E + I * E
        n_norm = {"SandwichBlock": 4}.get(self.block_class_name, 2)
        if self.norm_class_name not in ("Identity", "UnparametrizedRMSNorm"):
            per_block += n_norm * E
        if self.qk_bias:
            per_block += 2 * self.n_head * hd
        if self.is_recurrent:
            blocks = self.n_layers_in_prelude + self.n_layers_in_recurrent_block + self.n_layers_in_coda
            total = blocks * per_block + V * E + E
            if self.injection_type == "linear":
                total += 2 * E * E
            if not self.tie_embeddings:
                total += V * E
            return total
        return self.n_layer * per_block + 2 * V * E + E

    def flops_per_token(self, seq_len: int, n: int, k: int, checkpointing: bool = False) -> float:
        """Model FLOPs per token for a training step with ``n`` no-grad and ``k`` grad
        recurrences (2 FLOPs per multiply-add; causal attention counted at half)."""
        E, I, V = self.n_embd, self.intermediate_size, self.padded_vocab_size
        kv = self.num_key_value_heads * self.head_size
        gated = self.mlp_class_name.startswith("Gated")
        lin = (E + 2 * kv) * E + E * E + (3 if gated else 2) * I * E
        attn = 2 * seq_len * E / 2  # QK^T and PV, causal half
        block = 2 * (lin + attn)
        adapter = 2 * (2 * E * E) if self.injection_type == "linear" else 0
        head = 2 * V * E
        if not self.is_recurrent:
            return 3 * (self.n_layer * block + head)
        P, C, R = self.n_layers_in_prelude, self.n_layers_in_coda, self.n_layers_in_recurrent_block
        fwd = (P + C) * block + (n + k) * (R * block + adapter) + head
        bwd = 2 * ((P + C) * block + k * (R * block + adapter) + head)
        rec = k * (R * block + adapter) if checkpointing else 0
        return fwd + bwd + rec


# aliases that mirror the reference's class split (recpre/config_dynamic.py:354,392)
Config = ModelConfig
GPTConfig = ModelConfig
RecurrentConfig = ModelConfig
AnyConfig = ModelConfig


def sqrt_embd(cfg: ModelConfig) -> float:
    return math.sqrt(cfg.n_embd)
