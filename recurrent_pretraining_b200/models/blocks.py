"""Transformer building blocks selected by the string names used in model configs.

Parameter names (``norm_1..4.weight``, ``attn.Wqkv.weight``, ``attn.qk_bias``, ``attn.proj.weight``,
``mlp.fc.weight``, ``mlp.proj.weight``) and fused layouts (``Wqkv`` rows ``[Q;K;V]``, gated ``fc`` rows
``[gate;up]``) are the checkpoint contract of the reference (recpre/model_dynamic.py:150-412,745-780).
All arithmetic goes through ``ops.functional`` so the same module runs the PyTorch statements on CPU
and the sm_100a kernels on a GPU.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

import os

from ..ops import functional as ops

FUSE_SWIGLU = os.environ.get("B200_FUSE_SWIGLU", "1") == "1"
FUSE_ROPE = os.environ.get("B200_FUSE_ROPE", "1") == "1"


# ------------------------------------------------------------------------------------------
# primitives
# ------------------------------------------------------------------------------------------
class Linear(nn.Module):
    """Bias-optional linear layer whose weight is initialised by a role-aware initialiser
    (recpre/config_dynamic.py:450-467)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 init_method=None, init=None):
        """``init_method`` (the reference's keyword) or ``init``: callable that fills the weight in place; without one
        the weight is drawn from a normal of std 1/sqrt(in_features) truncated at three std (recpre/init.py:511-516)."""
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        self._init = init_method if init_method is not None else init
        self.reset_parameters()

    @property
    def init_method(self):
        return self._init

    def reset_parameters(self) -> None:
        if self._init is not None:
            self._init(self.weight)
        else:
            std = 1 / math.sqrt(self.in_features)
            nn.init.trunc_normal_(self.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, x, **kwargs):                  # extra arguments of tensor-parallel wrappers are ignored
        y = ops.linear(x, self.weight)
        return y if self.bias is None else y + self.bias.to(y.dtype)

    def extra_repr(self) -> str:
        return f"{self.in_features} -> {self.out_features}, bias={self.bias is not None}"


class RMSNorm(nn.Module):
    """RMS norm with a learned scale; statistics in fp32 (recpre/norms.py:19-75)."""

    def __init__(self, dim: int, eps: float = 1e-6, add_unit_offset: bool = False, learnable: bool = True):
        super().__init__()
        self.eps, self.add_unit_offset = eps, add_unit_offset
        self.weight = nn.Parameter(torch.ones(dim)) if learnable else None

    def _w(self):
        if self.weight is None:
            return None
        return 1 + self.weight if self.add_unit_offset else self.weight

    def forward(self, x):
        return ops.rmsnorm(x, self._w(), self.eps)

    def forward_add(self, a, x):
        """norm(a + x) in one pass."""
        return ops.add_rmsnorm(a, x, self._w(), self.eps)

    def reset_parameters(self) -> None:
        if self.weight is not None:
            nn.init.ones_(self.weight)


class _PlainNorm(nn.Module):
    """Adapter giving torch norms (LayerNorm / Identity) the ``forward_add`` entry."""

    def __init__(self, inner: nn.Module):
        super().__init__()
        self.inner = inner

    def forward(self, x):
        return self.inner(x)

    def forward_add(self, a, x):
        return self.inner(a + x)


class LayerNorm(nn.LayerNorm):
    def forward_add(self, a, x):
        return self.forward(a + x)


class Identity(nn.Identity):
    def __init__(self, *a, **k):
        super().__init__()

    def forward_add(self, a, x):
        return a + x


def make_norm(config, dim: int | None = None) -> nn.Module:
    dim = config.n_embd if dim is None else dim
    name = config.norm_class_name
    # every RMS form of the reference (recpre/norms.py:18-152: its own, the llama and gemma-like casts, torch's, the
    # Triton one) is the same function up to where the cast happens; here the statistics are always fp32
    if name in ("RMSNorm", "RMSNorm_llama", "FusedRMSNorm", "TorchRMSNorm", "GemmalikeRMS"):
        return RMSNorm(dim, eps=config.norm_eps, add_unit_offset="Gemma" in config.name)
    if name == "UnparametrizedRMSNorm":
        return RMSNorm(dim, eps=config.norm_eps, learnable=False)
    if name == "LayerNorm":
        return LayerNorm(dim, eps=config.norm_eps)
    if name == "OlmoLayerNorm":                      # layer norm without scale and shift
        return LayerNorm(dim, eps=config.norm_eps, elementwise_affine=False)
    if name == "Identity":
        return Identity()
    if hasattr(nn, name):                            # any other torch.nn norm by name, as the reference falls back to
        return _PlainNorm(getattr(nn, name)(dim, eps=config.norm_eps))
    raise ValueError(f"unknown norm class {name!r}")


class Relu2(nn.Module):
    """0.5 * relu(x)^2 (the factor is the reference's, recpre/config_dynamic.py:470-476)."""

    def __init__(self, inplace: bool = False):
        super().__init__()
        self.inplace = inplace

    def forward(self, x):
        return F.relu(x, inplace=self.inplace).square().mul(0.5)


def make_nonlin(name: str) -> nn.Module:
    if name == "ReLU2":
        return Relu2()
    if hasattr(nn, name):
        return getattr(nn, name)()
    raise ValueError(f"Could not identify nonlinearity {name}")


# ------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------
def _split_rope(qkv, qk_bias, cos, sin, n_head, n_kv, head_dim):
    """Differentiable unfused q/k/v path for the rarely used variants (qk_norm, telemetry, attention bypass)."""
    from ..ops import reference as ref

    return ref.qk_bias_rope(qkv, qk_bias, cos, sin, n_head, n_kv, head_dim)


def _dense_attention(q, k, v, softcap: float = 0.0):
    """fp32 statement of causal attention on [B,S,H,hd] tensors; ``softcap`` > 0 squashes the logits to
    ``softcap * tanh(logit / softcap)`` before the softmax (the ``flex-attention-soft-cap`` provider of the reference,
    recpre/attention_backends/flex_attentions.py:66-97, cap 20)."""
    from ..ops import reference as ref

    if softcap <= 0:
        return ref.causal_attention(q, k, v)
    B, S, H, D = q.shape
    Hk = k.shape[2]
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    if Hk != H:
        kf, vf = kf.repeat_interleave(H // Hk, dim=1), vf.repeat_interleave(H // Hk, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    return (torch.softmax(s, dim=-1) @ vf).transpose(1, 2).to(q.dtype).contiguous()


def _center_debias(y, v, n_head: int, center: bool, debias: bool):
    """Post-operations of the reference's attention providers on y, v as [B,S,H,hd] (recpre/attention_backends/
    pytorch.py:22-29): ``center`` adds the token's own value (attention matrix + identity), ``debias`` subtracts the
    causal running mean of the values (attention matrix - uniform causal attention)."""
    if v.shape[2] != n_head:
        v = v.repeat_interleave(n_head // v.shape[2], dim=2)
    if center:
        y = y + v
    if debias:
        S = y.shape[1]
        steps = torch.arange(1, S + 1, device=y.device, dtype=torch.float32)[None, :, None, None]
        y = y - (v.float().cumsum(dim=1) / steps).to(y.dtype)
    return y


class CausalSelfAttention(nn.Module):
    def __init__(self, config, layer_id: int):
        super().__init__()
        self.config = config
        self.n_head, self.n_kv = config.n_head, config.num_key_value_heads
        self.head_dim = config.n_embd // self.n_head
        width = (self.n_head + 2 * self.n_kv) * self.head_dim
        init = config.init
        self.Wqkv = Linear(config.n_embd, width, bias=config.bias,
                           init=lambda w: init.init_weight_(w, "qkv", layer_id))
        if config.qk_bias:
            self.qk_bias = nn.Parameter(torch.zeros(2, 1, self.n_head, self.head_dim))
        else:
            self.qk_bias = None
        self.proj = Linear(config.n_embd, config.n_embd, bias=config.bias,
                           init=lambda w: init.init_weight_(w, "out_attn", layer_id))
        self.layer_id = layer_id
        self.monitoring = False
        self.latest_metrics: dict = {}

    def forward(self, x, rope, mask=None):
        B, S, E = x.shape
        cos, sin = rope
        cfg = self.config
        post = cfg.center_attention or cfg.debias_attention
        softcap = 20.0 if cfg.attn_impl == "flex-attention-soft-cap" else 0.0
        plain = not (cfg.qk_norm or self.monitoring or cfg.attn_impl == "debug-skip" or softcap)
        # grouped keys with a q/k bias: the reference repeats k (and v) to all query heads and THEN adds the bias, which
        # has one row per query head (recpre/model_dynamic.py:357-366), so the keys differ inside a group
        expand = self.qk_bias is not None and self.n_kv != self.n_head
        n_kv = self.n_head if expand else self.n_kv
        if (plain and not post and not expand and FUSE_ROPE and x.is_cuda and self.config.clip_qkv is None and self.Wqkv.bias is None
                and self.config.rope_settings.use_rope):
            # bias + rotation ride in the epilogue of the QKV GEMM
            y = ops.qkv_rope_attention(x, self.Wqkv.weight, self.qk_bias, cos, sin, self.n_head, self.n_kv, self.head_dim)
            return self.proj(y)
        qkv = self.Wqkv(x)
        if self.config.clip_qkv is not None:
            qkv = qkv.clamp(min=-self.config.clip_qkv, max=self.config.clip_qkv)
        if expand:
            wq, wk, rep = self.n_head * self.head_dim, self.n_kv * self.head_dim, self.n_head // self.n_kv
            q, k, v = qkv.split([wq, wk, wk], dim=-1)
            k, v = (t.reshape(B, S, self.n_kv, 1, self.head_dim).expand(B, S, self.n_kv, rep, self.head_dim)
                    .reshape(B, S, wq) for t in (k, v))
            qkv = torch.cat([q, k, v], dim=-1)
        if not self.config.rope_settings.use_rope:
            cos, sin = torch.ones_like(cos), torch.zeros_like(sin)
        if plain:
            y = ops.rope_attention(qkv, self.qk_bias, cos, sin, self.n_head, n_kv, self.head_dim)
            if post:     # the providers' post-operations need the (un-rotated) values beside the attention output
                wq, wk = self.n_head * self.head_dim, n_kv * self.head_dim
                v = qkv[..., wq + wk:].reshape(B, S, n_kv, self.head_dim)
                y = _center_debias(y.reshape(B, S, self.n_head, self.head_dim), v, self.n_head, cfg.center_attention,
                                   cfg.debias_attention).reshape(B, S, E)
            return self.proj(y)
        q, k, v = _split_rope(qkv, self.qk_bias, cos, sin, self.n_head, n_kv, self.head_dim)
        if self.config.qk_norm:
            q = F.rms_norm(q, (q.shape[-1],))
            k = F.rms_norm(k, (k.shape[-1],))
        if self.config.attn_impl == "debug-skip":
            # attention bypass for pure-GEMM sanity models: the values pass through (recpre/attention_backends/
            # interface.py:37-39)
            y = v if n_kv == self.n_head else v.repeat_interleave(self.n_head // n_kv, dim=2)
        else:
            y = _dense_attention(q, k, v, softcap)
            if post:
                y = _center_debias(y, v, self.n_head, cfg.center_attention, cfg.debias_attention)
        if self.monitoring:
            self._monitor(q, k)
        return self.proj(y.reshape(B, S, E))

    def monitor_layer(self, q, k, mask=None):
        """The reference's name for the attention telemetry (q, k as [B, S, H, hd])."""
        self._monitor(q, k)
        return self.latest_metrics

    @torch.no_grad()
    def _monitor(self, q, k):
        """Attention-entropy / max-logit telemetry on a small slice (recpre/model_dynamic.py:389-412)."""
        qs, ks = q[:1, :256].float().transpose(1, 2), k[:1, :256].float().transpose(1, 2)
        if ks.shape[1] != qs.shape[1]:
            ks = ks.repeat_interleave(qs.shape[1] // ks.shape[1], dim=1)
        logits = qs @ ks.transpose(-1, -2) / math.sqrt(q.shape[-1])
        S = logits.shape[-1]
        logits = logits.masked_fill(torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
        p = torch.softmax(logits, dim=-1)
        ent = -(p * torch.log(p.clamp_min(1e-30))).sum(-1).mean()
        self.latest_metrics = {f"attn_entropy_{self.layer_id}": ent.item(),
                               f"max_attn_logit_{self.layer_id}": logits[logits.isfinite()].max().item()}


# ------------------------------------------------------------------------------------------
# MLPs
# ------------------------------------------------------------------------------------------
class BaseMLP(nn.Module):
    def __init__(self, config, layer_id: int = 0, in_features: int = 0):
        super().__init__()
        in_features = in_features or config.n_embd
        init = config.init
        self.fc = Linear(in_features, config.intermediate_size, bias=config.bias,
                         init=lambda w: init.init_weight_(w, "in_proj", layer_id))
        self.proj = Linear(config.intermediate_size, config.n_embd, bias=config.bias,
                           init=lambda w: init.init_weight_(w, "out_proj", layer_id))
        self.nonlin = make_nonlin(config.nonlin_name)

    def forward(self, x):
        return self.proj(self.nonlin(self.fc(x)))


class GatedMLP(nn.Module):
    """proj(nonlin(gate) * up) with a single fused ``fc`` producing [gate | up]."""

    def __init__(self, config, layer_id: int = 0, in_features: int = 0):
        super().__init__()
        in_features = in_features or config.n_embd
        init = config.init
        self.fc = Linear(in_features, 2 * config.intermediate_size, bias=config.bias,
                         init=lambda w: init.init_weight_(w, "glu", layer_id))
        self.proj = Linear(config.intermediate_size, config.n_embd, bias=config.bias,
                           init=lambda w: init.init_weight_(w, "out_proj", layer_id))
        self.is_silu = config.nonlin_name == "SiLU"
        self.nonlin = make_nonlin(config.nonlin_name)

    def forward(self, x):
        if self.is_silu and self.fc.bias is None and x.is_cuda and not torch.is_grad_enabled() and FUSE_SWIGLU:
            return self.proj(ops.linear_swiglu(x, self.fc.weight))  # gate applied in the GEMM epilogue
        if self.is_silu and self.fc.bias is None and self.proj.bias is None and x.is_cuda and FUSE_SWIGLU \
                and torch.is_grad_enabled() and type(self.proj) is Linear:   # a row-parallel proj reduces in its forward
            return ops.gated_mlp(x, self.fc.weight, self.proj.weight)   # both elementwise stages in GEMM epilogues
        h = self.fc(x)
        if self.is_silu:
            return self.proj(ops.swiglu(h))
        a, b = h.chunk(2, dim=-1)
        return self.proj(self.nonlin(a) * b)


class BrickLP(nn.Module):
    def __init__(self, config, layer_id: int = 0, in_features: int = 0):
        super().__init__()
        in_features = in_features or config.n_embd
        self.fc = Linear(in_features, in_features, bias=False)

    def forward(self, x):
        return self.fc(x)


MLP_CLASSES = {"BaseMLP": BaseMLP, "GatedMLP": GatedMLP, "LLaMAMLP": GatedMLP, "BrickLP": BrickLP}


def make_mlp(config, layer_id: int, in_features: int = 0) -> nn.Module:
    try:
        return MLP_CLASSES[config.mlp_class_name](config, layer_id, in_features)
    except KeyError:
        raise ValueError(f"unknown MLP class {config.mlp_class_name!r}") from None


# ------------------------------------------------------------------------------------------
# blocks
# ------------------------------------------------------------------------------------------
class _TwoNormBlock(nn.Module):
    expanded = False

    def __init__(self, config, layer_id: int):
        super().__init__()
        self.config, self.layer_id = config, layer_id
        self.norm_1 = make_norm(config)
        self.attn = CausalSelfAttention(config, layer_id)
        self.norm_2 = make_norm(config)
        self.mlp = make_mlp(config, layer_id)
        res, skip = config.init.get_scales(layer_id)
        self.register_buffer("res_scale", torch.as_tensor(res), persistent=True)
        self.register_buffer("skip_scale", torch.as_tensor(skip), persistent=True)


class TransformerScaledPreNormBlock(_TwoNormBlock):
    def forward(self, x, rope, mask=None):
        x = self.attn(self.norm_1(x), rope, mask) * self.res_scale + x * self.skip_scale
        return self.mlp(self.norm_2(x)) * self.res_scale + x * self.skip_scale


class TransformerPreNormBlock(_TwoNormBlock):
    def forward(self, x, rope, mask=None):
        x = self.attn(self.norm_1(x), rope, mask) + x
        return self.mlp(self.norm_2(x)) + x


class TransformerPostNormBlock(_TwoNormBlock):
    def forward(self, x, rope, mask=None):
        x = self.norm_1.forward_add(self.attn(x, rope, mask), x)
        return self.norm_2.forward_add(self.mlp(x), x)


class ScaledTransformerPostNormBlock(_TwoNormBlock):
    def forward(self, x, rope, mask=None):
        x = self.norm_1(self.attn(x, rope, mask) * self.res_scale + x * self.skip_scale)
        return self.norm_2(self.mlp(x) * self.res_scale + x * self.skip_scale)


class SwinBlock(_TwoNormBlock):
    def forward(self, x, rope, mask=None):
        x = self.norm_1(self.attn(x, rope, mask)) + x
        return self.norm_2(self.mlp(x)) + x


class SandwichBlock(nn.Module):
    """x = n2(attn(n1(x)) + x); x = n4(mlp(n3(x)) + x)   (recpre/model_dynamic.py:265-288)."""

    expanded = False

    def __init__(self, config, layer_id: int):
        super().__init__()
        self.config, self.layer_id = config, layer_id
        self.norm_1 = make_norm(config)
        self.attn = CausalSelfAttention(config, layer_id)
        self.norm_2 = make_norm(config)
        self.norm_3 = make_norm(config)
        self.mlp = make_mlp(config, layer_id)
        self.norm_4 = make_norm(config)

    def forward(self, x, rope, mask=None):
        x = self.norm_2.forward_add(self.attn(self.norm_1(x), rope, mask), x)
        return self.norm_4.forward_add(self.mlp(self.norm_3(x)), x)


class Brick(nn.Module):
    expanded = False

    def __init__(self, config, layer_id: int):
        super().__init__()
        self.mlp = make_mlp(config, layer_id)
        self.layer_id = layer_id

    def forward(self, x, rope, mask=None):
        return self.mlp(x)


BLOCK_CLASSES = {c.__name__: c for c in (
    TransformerScaledPreNormBlock, TransformerPreNormBlock, TransformerPostNormBlock,
    ScaledTransformerPostNormBlock, SwinBlock, SandwichBlock, Brick)}


def make_block(config, layer_id: int) -> nn.Module:
    try:
        return BLOCK_CLASSES[config.block_class_name](config, layer_id)
    except KeyError:
        raise ValueError(f"unknown block class {config.block_class_name!r}") from None
