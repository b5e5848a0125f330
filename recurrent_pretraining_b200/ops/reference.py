"""Plain PyTorch statements of every op the framework uses.

These are the numerical oracles for the CUDA kernels (tests compare a kernel against the
function of the same name evaluated in fp32) and the execution path on CPU.  Each function
names the reference behaviour it restates.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """y = cast_x(x32 * rsqrt(mean(x32^2) + eps)) * w   (recpre/norms.py:63-68).  The output keeps the
    dtype of ``x`` (the framework carries a bf16 residual stream on GPU)."""
    x32 = x.float()
    y = x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y.to(x.dtype).float() * weight.float()
    return y.to(x.dtype)


def add_rmsnorm(a: torch.Tensor, x: torch.Tensor, weight: torch.Tensor | None, eps: float) -> torch.Tensor:
    """Sandwich post-norm: norm(a + x) where the sum is rounded to the stream dtype first
    (recpre/model_dynamic.py:279-282)."""
    return rmsnorm((a.float() + x.float()).to(x.dtype), weight, eps)


def rope_tables(head_dim: int, length: int, base: float = 50000.0, condense: int = 1) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables [length, head_dim/2] in fp32 (recpre/model_dynamic.py:1438-1443)."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    t = torch.arange(length, dtype=torch.float32) / condense
    ang = torch.outer(t, inv).float()
    return torch.cos(ang), torch.sin(ang)


def freqs_cis_buffer(cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """The state-dict form ``[1, S, 1, hd/2, 2]`` of the tables."""
    return torch.stack([cos[None, :, None, :], sin[None, :, None, :]], dim=4)


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate interleaved pairs (2i, 2i+1) of the last dim of ``x`` [B,S,H,hd]; cos/sin are [S, hd/2] (or
    broadcastable [B,S,1,hd/2]); math in fp32, result in x.dtype (recpre/model_dynamic.py:1450-1462)."""
    if cos.ndim == 2:
        cos, sin = cos[None, :, None, :], sin[None, :, None, :]
    xr = x.float().unflatten(-1, (-1, 2))
    a, b = xr[..., 0], xr[..., 1]
    out = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    return out.to(x.dtype)


def qk_bias_rope(qkv: torch.Tensor, qk_bias: torch.Tensor | None, cos: torch.Tensor, sin: torch.Tensor,
                 n_head: int, n_kv: int, head_dim: int):
    """Split fused qkv [B,S,(H+2Hkv)*hd] into q,k,v [B,S,H,hd], add the q/k bias, rotate q and k
    (recpre/model_dynamic.py:349-370)."""
    B, S, _ = qkv.shape
    q, k, v = qkv.split([n_head * head_dim, n_kv * head_dim, n_kv * head_dim], dim=-1)
    q = q.reshape(B, S, n_head, head_dim)
    k = k.reshape(B, S, n_kv, head_dim)
    v = v.reshape(B, S, n_kv, head_dim)
    if qk_bias is not None:
        q = (q.float() + qk_bias[0].float()).to(qkv.dtype)
        k = (k.float() + qk_bias[1].float()).to(qkv.dtype)
    return rope_interleaved(q, cos, sin), rope_interleaved(k, cos, sin), v.contiguous()


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None,
                     q_offset: int = 0) -> torch.Tensor:
    """softmax(q k^T * scale + causal) v with q,k,v as [B,S,H,hd]; returns [B,Sq,H,hd].  ``q_offset`` is the
    absolute position of the first query row (for cached decode, keys start at position 0)."""
    B, Sq, H, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    if Hk != H:
        kf = kf.repeat_interleave(H // Hk, dim=1)
        vf = vf.repeat_interleave(H // Hk, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    qi = torch.arange(Sq, device=q.device)[:, None] + q_offset
    ki = torch.arange(Sk, device=q.device)[None, :]
    s = s.masked_fill(ki > qi, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf).transpose(1, 2).to(q.dtype).contiguous()


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor,
                     scale: float | None = None) -> torch.Tensor:
    """softmax(q k^T * scale, restricted to ``mask``) v with q,k,v as [B,S,H,hd] and a boolean ``mask`` [B,1,Sq,Sk]
    (True = may attend).  A query row that may attend to nothing (a padding position) returns zeros."""
    B, Sq, H, D = q.shape
    Hk = k.shape[2]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    if Hk != H:
        kf = kf.repeat_interleave(H // Hk, dim=1)
        vf = vf.repeat_interleave(H // Hk, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.matmul(p, vf).transpose(1, 2).to(q.dtype).contiguous()


def swiglu(h: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up with ``h = [gate | up]`` along the last dim (recpre/model_dynamic.py:776-780)."""
    a, b = h.float().chunk(2, dim=-1)
    return (F.silu(a) * b).to(h.dtype)


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return F.linear(x, w.to(x.dtype))


def adapter(x: torch.Tensor, e: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Linear(2E -> E) on cat[state, embedding] (recpre/model_dynamic.py:1210)."""
    return F.linear(torch.cat([x, e.to(x.dtype)], dim=-1), w.to(x.dtype))


def embedding(ids: torch.Tensor, w: torch.Tensor, scale: float) -> torch.Tensor:
    return F.embedding(ids, w) * scale


def linear_cross_entropy(x: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, logit_scale: float = 1.0,
                         ignore_index: int = -100, z_reg: float = 0.0) -> torch.Tensor:
    """mean over valid rows of CE(float(x w^T) * logit_scale, label) (+ z_reg * lse^2), the quantities of
    recpre/ops.py:12-20 and recpre/model_dynamic.py:1133-1134."""
    logits = F.linear(x, w.to(x.dtype)).float() * logit_scale
    flat = logits.view(-1, logits.shape[-1])
    lab = labels.reshape(-1)
    loss = F.cross_entropy(flat, lab, ignore_index=ignore_index)
    if z_reg:
        valid = lab != ignore_index
        lse = torch.logsumexp(flat, dim=-1)
        loss = loss + z_reg * (lse.pow(2) * valid).sum() / valid.sum().clamp(min=1)
    return loss


def trunc_normal_state(shape, std: float, generator: torch.Generator | None = None, device="cpu",
                       dtype=torch.float32) -> torch.Tensor:
    """State init: normal(0, std) truncated at +-3 std (recpre/model_dynamic.py:1360-1365)."""
    x = torch.empty(shape, dtype=torch.float32, device=device)
    torch.nn.init.trunc_normal_(x, mean=0.0, std=std, a=-3 * std, b=3 * std, generator=generator)
    return x.to(dtype)


def adamw_step(p, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    """Decoupled-weight-decay Adam on fp32 tensors, in place (torch.optim.AdamW semantics)."""
    g = g * grad_scale
    p.mul_(1 - lr * wd)
    m.lerp_(g, 1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
