"""Parameter grouping by name (recpre/optim.py:18-56): weights / embeddings / scales-norms-biases.

Group order is part of the contract: the ZeRO-style shard rule and the checkpointed optimizer state index
groups positionally.  ``qk_bias`` lands in the norm group because its name contains "bias".
"""
from __future__ import annotations


def classify(name: str, ndim: int) -> str:
    l = name.lower()
    if "wte" in l or "embedding" in l or "abacus" in l or "lm_head" in l:
        return "embedding"
    if "ln_f" in l or "norm" in l or "bias" in l or "diff_lmb" in name:
        return "norm"
    if "proj" in l or "qkv" in l or "fc" in l or ndim == 2:
        return "weight"
    raise ValueError(f"param {name} could not be matched to an optimizer group")


def get_param_groups(named_parameters, no_weight_decay_for_bias_and_norm_params: bool = True,
                     weight_lr_scale: float = 1.0, no_wd_on_embedding: bool = False, verbose: bool = False,
                     with_names: bool = False):
    buckets = {"weight": [], "embedding": [], "norm": []}
    names = {"weight": [], "embedding": [], "norm": []}
    for name, p in named_parameters:
        kind = classify(name, p.ndim)
        if verbose:
            print(f"Matched {name} to the {kind} group")
        buckets[kind].append(p)
        names[kind].append(name)
    groups = [
        {"params": buckets["weight"], "base_lr": weight_lr_scale},
        {"params": buckets["embedding"], "base_lr": 1.0},
        {"params": buckets["norm"], "base_lr": 1.0},
    ]
    if no_wd_on_embedding:
        groups[1]["weight_decay"] = 0.0
    if no_weight_decay_for_bias_and_norm_params:
        groups[2]["weight_decay"] = 0.0
    if with_names:
        for g, k in zip(groups, ("weight", "embedding", "norm")):
            g["names"] = names[k]
    return groups
