"""Optimizer lookup by name (recpre/optim.py:59-128): any ``torch.optim`` class, the named research optimizers, the two
external ones when their packages are installed (apex ``FusedAdam``, Meta's distributed Shampoo), ``fused=True`` for
every class that offers it, and optional ZeRO-1-style sharding of optimizer state over the ranks."""
from __future__ import annotations

import inspect
from functools import partial

import torch


def get_optimizer(optimizer_name: str, model=None, pytorch_optimizer_sharding: bool = False,
                  allow_fusion: bool = True, use_apex_adamw: bool = False, use_zero: bool = False):
    name = optimizer_name
    if hasattr(torch.optim, name):
        cls = getattr(torch.optim, name)
    elif name == "LionW":
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
    elif name == "meta-shampoo":
        try:
            from distributed_shampoo.distributed_shampoo import DistributedShampoo
            from distributed_shampoo.shampoo_types import AdamGraftingConfig, CommunicationDType, DDPShampooConfig
        except ModuleNotFoundError:
            raise ValueError("Invalid optimizer meta-shampoo requested: the distributed_shampoo package is not "
                             "installed ('simo-shampoo' is the built-in blocked Shampoo)") from None
        cls = partial(DistributedShampoo, grafting_config=AdamGraftingConfig(beta2=0.95, epsilon=1e-8),
                      distributed_config=DDPShampooConfig(communication_dtype=CommunicationDType.FP32,
                                                          num_trainers_per_group=max(torch.cuda.device_count(), 1),
                                                          communicate_params=False))
    else:
        raise ValueError(f"Invalid optimizer {name} requested.")
    if name == "AdamW" and use_apex_adamw:
        try:
            from apex.optimizers import FusedAdam as cls
        except ModuleNotFoundError:
            raise ValueError("Need to install apex!") from None
    if allow_fusion and torch.cuda.is_available():
        target = cls.func if isinstance(cls, partial) else cls
        if "fused" in inspect.signature(target).parameters:       # every optimizer class that offers a fused kernel
            cls = partial(cls, fused=True)
    if use_zero or (pytorch_optimizer_sharding and torch.distributed.is_available()
                    and torch.distributed.is_initialized()):
        from .zero import SimpleZeroRedundancyOptimizer

        return partial(SimpleZeroRedundancyOptimizer, optimizer_class=cls)
    return cls
