"""Optimizer lookup by name (recpre/optim.py:59-128): any ``torch.optim`` class, the named research optimizers, and
optional ZeRO-1-style sharding of optimizer state over the ranks of a node."""
from __future__ import annotations

from functools import partial

import torch


def get_optimizer(optimizer_name: str, model=None, pytorch_optimizer_sharding: bool = False,
                  allow_fusion: bool = True, use_apex_adamw: bool = False, use_zero: bool = False):
    name = optimizer_name
    if name == "LionW":
        from .others import LionW as cls
    elif name == "SophiaG":
        from .others import SophiaG as cls
    elif name == "ELLISAdam":
        from .ellis import ELLISAdam as cls
    elif name == "SOAP":
        from .soap import SOAP as cls
    elif name == "Lilith":
        from .research import Lilith as cls
    elif name == "IVON":
        from .research import IVON as cls
    elif name in ("simo-shampoo", "ZeroShampoo", "ZeroShampooWithAdamGraftingOptimizer"):
        from .research import ZeroShampooWithAdamGraftingOptimizer as cls
    elif name in ("Kellers", "OrthogonalNesterov"):
        from .others import OrthogonalNesterov as cls
    elif hasattr(torch.optim, name):
        cls = getattr(torch.optim, name)
        if allow_fusion and name in ("AdamW", "Adam", "SGD") and torch.cuda.is_available():
            cls = partial(cls, fused=True)
    else:
        raise ValueError(f"Invalid optimizer {name} requested (meta's distributed_shampoo package is not bundled).")
    if use_zero or pytorch_optimizer_sharding:
        from .zero import SimpleZeroRedundancyOptimizer

        return partial(SimpleZeroRedundancyOptimizer, optimizer_class=cls)
    return cls
