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
