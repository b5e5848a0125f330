"""The earlier Hub-facing model file, kept for checkpoints and scripts that were written against it.

What differs from the current inference model, as in the reference (recpre/legacy_modeling_file.py:219-267, 395-447):
the attention of every block can run "eagerly" (explicit softmax) and return its attention map, collected per KV-cache
step index in ``output.attention_maps`` when ``output_details["return_attention"]`` is set.  Everything else (config,
cache, generation) is the current implementation under the names the old file exported.
"""
from __future__ import annotations

import math

import torch

from ..ops import functional as ops
from . import hf as _hf
from .hf_config import RavenConfig  # noqa: F401  (re-exported)
from .kv_cache import RecurrentKVCache

HuginnDynamicCache = RecurrentKVCache
CausalLMOutputRecurrentLatents = _hf.CausalLMOutputRecurrentLatents
RavenPreTrainedModel = _hf.RavenPreTrainedModel


def eager_causal_attention(q, k, v, offset: int):
    """q [B,Sq,H,D], k/v [B,Sk,Hkv,D]; returns (y [B,Sq,H,D], map [B,Sq,Sk]) where the map is the maximum over heads of
    the attention weights."""
    if k.shape[2] != q.shape[2]:
        rep = q.shape[2] // k.shape[2]
        k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
    qh, kh, vh = (t.transpose(1, 2).float() for t in (q, k, v))
    scores = qh @ kh.transpose(-1, -2) / math.sqrt(q.shape[-1])
    Sq, Sk = scores.shape[-2:]
    if Sq > 1:
        rows = torch.arange(Sq, device=q.device)[:, None] + offset
        scores = scores.masked_fill(torch.arange(Sk, device=q.device)[None, :] > rows, float("-inf"))
    w = torch.softmax(scores, dim=-1)
    return (w @ vh).transpose(1, 2).to(q.dtype), w.max(dim=1)[0]


class RavenForCausalLM(_hf.RavenForCausalLM):
    _collect_maps = None

    def _attention(self, attn, x, rope, step_idx: int, cache):
        if self._collect_maps is None:
            return super()._attention(attn, x, rope, step_idx, cache)
        B, S, E = x.shape
        cos, sin = rope
        q, k, v = ops.qk_bias_rope(attn.Wqkv(x), attn.qk_bias, cos, sin, attn.n_head, attn.n_kv, attn.head_dim)
        if cache is not None:
            k, v = cache.update(k, v, step_idx)
        y, amap = eager_causal_attention(q, k, v, k.shape[1] - q.shape[1])
        self._collect_maps[step_idx] = amap
        return attn.proj(y.reshape(B, S, E))

    def forward(self, *args, output_details: dict | None = None, **kwargs):
        details = dict(_hf._DEFAULT_DETAILS, **(output_details or {}))
        want = bool(details.pop("return_attention", False))
        self._collect_maps = {} if want else None
        try:
            out = super().forward(*args, output_details=details, **kwargs)
            if want:
                out["attention_maps"] = self._collect_maps
        finally:
            self._collect_maps = None
        return out

    # -- older signatures ---------------------------------------------------------------------------
    def initialize_state(self, input_embeds, deterministic=False, scale: float = 1.0):
        """The old file took ``deterministic`` (True: an all-zero state) where the current one takes ``scale``
        (recpre/legacy_modeling_file.py:620-626); both spellings are accepted here."""
        if isinstance(deterministic, (int, float)) and not isinstance(deterministic, bool):
            scale, deterministic = float(deterministic), False      # positional ``scale`` of the current API
        if deterministic:
            return torch.zeros_like(input_embeds)
        return super().initialize_state(input_embeds, scale)

    def compute_eager_sdpa(self, q, k, v, attn_mask=None):
        """[B, H, S, D] operands, explicit softmax; returns (y, attention map maxed over heads), as the old file's
        attention did when maps were requested (recpre/legacy_modeling_file.py:255-267)."""
        y, amap = eager_causal_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                         k.shape[2] - q.shape[2])
        return y.transpose(1, 2), amap

    def get_stats(self, logits, x, latent_states, xk, input_embeds, num_steps_no_grad, num_steps_with_grad):
        """Entropy of the prediction and (relative) distance between the last two latent states per position."""
        probs = torch.softmax(logits.float(), dim=-1)
        entropy = torch.where(probs > 0, -probs * probs.log(), torch.zeros_like(probs)).sum(dim=-1)
        diff = (x - latent_states).norm(dim=-1)
        return {"entropy": entropy, "residual_diff": diff, "rel_residual": diff / latent_states.norm(dim=-1),
                "num_steps_no_grad": num_steps_no_grad, "num_steps_with_grad": num_steps_with_grad}


def precompute_freqs_cis(dim: int, end: int, theta: float = 10000.0, condense_ratio: int = 1):
    """cos / sin table ``[1, end, 1, dim / 2, 2]`` in fp32 (module-level helper of the old file)."""
    from ..ops import reference as ref

    cos, sin = ref.rope_tables(dim, end, theta, condense_ratio)
    return ref.freqs_cis_buffer(cos, sin)


def apply_rotary_emb_complex_like(q, k, freqs_cis):
    """Rotate q and k ``[B, S, H, D]`` with a table from ``precompute_freqs_cis`` (already cut to S positions)."""
    from ..ops import reference as ref

    cos, sin = freqs_cis[0, :, 0, :, 0], freqs_cis[0, :, 0, :, 1]
    return ref.rope_interleaved(q, cos, sin), ref.rope_interleaved(k, cos, sin)


def register_auto_classes() -> None:
    """``AutoConfig`` / ``AutoModel`` / ``AutoModelForCausalLM`` registration under ``huginn_raven`` (the old file did
    this at import; here it is explicit because the current model file registers the same names)."""
    from transformers import AutoConfig, AutoModel, AutoModelForCausalLM

    for reg, args in ((AutoConfig, ("huginn_raven", RavenConfig)), (AutoModel, (RavenConfig, RavenForCausalLM)),
                      (AutoModelForCausalLM, (RavenConfig, RavenForCausalLM))):
        try:
            reg.register(*args, exist_ok=True)
        except TypeError:
            try:
                reg.register(*args)
            except ValueError:
                pass


# block classes of the old file, by their old names
def __getattr__(name: str):
    from . import blocks

    table = {"RMSNorm": blocks.RMSNorm, "CausalSelfAttention": blocks.CausalSelfAttention,
             "GatedMLP": getattr(blocks, "GatedMLP", None), "SandwichBlock": getattr(blocks, "SandwichBlock", None)}
    if name in table and table[name] is not None:
        return table[name]
    raise AttributeError(name)
