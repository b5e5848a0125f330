"""One-dimensional tensor parallelism for the transformer blocks (Megatron-style column / row split).

The reference reaches tensor parallelism only through the external AxoNN package (`axonn.intra_layer.Linear`,
recpre/config_dynamic.py:183-191, train.py:147-156), which is not installed and not used by its shipped runs.  This
module gives the same capability natively for a single node: attention heads and MLP channels are split over the
ranks of a process group; every block needs two all-reduces in the forward pass (after the attention output
projection and after the MLP output projection) and two in the backward pass (at the inputs of the two sub-layers).

    group = dist.new_group(ranks)                       # or None for the world
    tensor_parallelize(model, group)                    # shards the block weights in place (keeps this rank's part)

All other parameters (embedding, norms, adapter, head) stay replicated; their gradients are identical on every rank.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models import blocks as B


class _CopyToGroup(torch.autograd.Function):
    """Identity in the forward pass, all-reduce of the gradient in the backward pass (input of a column-parallel layer)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromGroup(torch.autograd.Function):
    """All-reduce in the forward pass, identity in the backward pass (output of a row-parallel layer)."""

    @staticmethod
    def forward(ctx, y, group):
        y = y.contiguous()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class RowParallelLinear(B.Linear):
    """Linear whose input channels are split over the group: each rank multiplies its slice, the partial results are
    summed.  A bias (if any) is added after the reduction by rank-independent code."""

    def __init__(self, weight_shard: torch.Tensor, bias, group):
        nn.Module.__init__(self)
        self.out_features, self.in_features = weight_shard.shape
        self.weight = nn.Parameter(weight_shard.clone())
        self.bias = bias
        self._init = None
        self.group = group

    def forward(self, x):
        y = _ReduceFromGroup.apply(B.ops.linear(x, self.weight), self.group)
        return y if self.bias is None else y + self.bias.to(y.dtype)


class TPCausalSelfAttention(B.CausalSelfAttention):
    def forward(self, x, rope, mask=None):
        return super().forward(_CopyToGroup.apply(x, self.tp_group), rope, mask)


class TPGatedMLP(B.GatedMLP):
    def forward(self, x):
        return super().forward(_CopyToGroup.apply(x, self.tp_group))


def _rank_size(group):
    return dist.get_rank(group), dist.get_world_size(group)


def shard_attention(attn: B.CausalSelfAttention, group) -> None:
    """Keep this rank's heads: rows of the fused [Q; K; V] projection, the q/k bias, and the matching input columns of
    the output projection (which becomes row-parallel)."""
    rank, tp = _rank_size(group)
    H, Hkv, D = attn.n_head, attn.n_kv, attn.head_dim
    assert H % tp == 0 and Hkv % tp == 0, "head counts must divide by the tensor-parallel size"
    h, hk = H // tp, Hkv // tp
    W = attn.Wqkv.weight.data
    E = W.shape[1]
    wq, wk = H * D, Hkv * D
    q = W[:wq].view(H, D, E)[rank * h:(rank + 1) * h].reshape(h * D, E)
    k = W[wq:wq + wk].view(Hkv, D, E)[rank * hk:(rank + 1) * hk].reshape(hk * D, E)
    v = W[wq + wk:].view(Hkv, D, E)[rank * hk:(rank + 1) * hk].reshape(hk * D, E)
    shard = B.Linear(E, (h + 2 * hk) * D, bias=False)
    shard.weight = nn.Parameter(torch.cat([q, k, v], 0).clone())
    if attn.Wqkv.bias is not None:
        raise NotImplementedError("tensor parallel attention with a projection bias")
    attn.Wqkv = shard
    if attn.qk_bias is not None:
        attn.qk_bias = nn.Parameter(attn.qk_bias.data[:, :, rank * h:(rank + 1) * h].clone())
    pw = attn.proj.weight.data
    attn.proj = RowParallelLinear(pw[:, rank * h * D:(rank + 1) * h * D], attn.proj.bias, group)
    attn.n_head, attn.n_kv = h, hk
    attn.tp_group = group
    attn.__class__ = TPCausalSelfAttention


def shard_gated_mlp(mlp: B.GatedMLP, group) -> None:
    """Keep this rank's slice of the hidden channels: the same rows of the gate and of the up half of ``fc`` and the
    matching input columns of ``proj``."""
    rank, tp = _rank_size(group)
    W = mlp.fc.weight.data
    I = W.shape[0] // 2
    assert I % tp == 0, "intermediate size must divide by the tensor-parallel size"
    i = I // tp
    shard = B.Linear(W.shape[1], 2 * i, bias=False)
    shard.weight = nn.Parameter(torch.cat([W[rank * i:(rank + 1) * i], W[I + rank * i:I + (rank + 1) * i]], 0).clone())
    if mlp.fc.bias is not None:
        raise NotImplementedError("tensor parallel MLP with a projection bias")
    mlp.fc = shard
    mlp.proj = RowParallelLinear(mlp.proj.weight.data[:, rank * i:(rank + 1) * i], mlp.proj.bias, group)
    mlp.tp_group = group
    mlp.__class__ = TPGatedMLP


def tensor_parallelize(model: nn.Module, group=None) -> nn.Module:
    """Shard every attention and gated-MLP module of ``model`` in place over ``group`` (default: all ranks)."""
    for m in list(model.modules()):
        if type(m) is B.CausalSelfAttention:
            shard_attention(m, group)
        elif type(m) is B.GatedMLP:
            shard_gated_mlp(m, group)
    return model


def gather_full_weight(param_shard: torch.Tensor, group=None, dim: int = 0) -> torch.Tensor:
    """All-gather a sharded tensor along ``dim`` (for checkpoints written in the unsharded layout)."""
    parts = [torch.empty_like(param_shard) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, param_shard.contiguous(), group=group)
    return torch.cat(parts, dim)
