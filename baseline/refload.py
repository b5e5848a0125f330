"""Import the *unmodified* reference package from ``baseline/_ref`` in an environment that lacks some of its
optional dependencies.

Nothing in the reference tree is edited.  The loader only (a) registers a bare ``recpre`` package object so
that ``recpre/__init__.py`` (which imports lightning, lm-eval glue and the HF model eagerly) is not executed,
(b) installs empty stand-ins for modules the reference imports at module top but does not need for its model,
optimiser and all-reduce code (``lightning``, ``torchmetrics``, ``jsonargparse``, ``axonn``, ``wandb``), and
(c) supplies one symbol that the reference imports from a private torch module and that torch 2.11 dropped.
Used as the numerical oracle in tests and as the ``--impl reference`` arm of ``bench.py``.
"""
from __future__ import annotations

import importlib
import importlib.machinery
import os
import sys
import types

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(_HERE, "_ref")


def available() -> bool:
    return os.path.isdir(os.path.join(REF_ROOT, "recpre"))


class _Anything:
    """Attribute sink: any attribute access or call returns another sink."""

    def __init__(self, *a, **k):
        pass

    def __getattr__(self, name):
        if name.startswith("__") and name.endswith("__"):
            raise AttributeError(name)
        return _Anything

    def __call__(self, *a, **k):
        return _Anything()


class _StubModule(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__") and name.endswith("__"):
            raise AttributeError(name)
        cls = type(name, (_Anything,), {})
        setattr(self, name, cls)
        return cls


_STUBS = [
    "lightning", "lightning.fabric", "lightning.fabric.strategies", "lightning.fabric.utilities",
    "lightning.fabric.utilities.load", "lightning.fabric.utilities.apply_func", "lightning.fabric.utilities.throughput",
    "lightning.fabric.utilities.rank_zero", "lightning.fabric.utilities.types", "lightning.fabric.loggers",
    "lightning.fabric.wrappers", "lightning.fabric.plugins", "lightning.fabric.plugins.environments",
    "lightning.fabric.strategies.fsdp", "lightning.pytorch", "lightning.pytorch.loggers",
    "lightning.pytorch.utilities", "lightning.pytorch.utilities.types", "lightning.pytorch.cli",
    "lightning_utilities", "lightning_utilities.core", "lightning_utilities.core.imports",
    "torchmetrics", "torchmetrics.aggregation", "jsonargparse", "axonn", "axonn.intra_layer", "axonn.lightning",
    "wandb", "torchdata", "torchdata.stateful_dataloader", "cut_cross_entropy", "lm_eval",
]


def _install_stubs() -> None:
    for name in _STUBS:
        if name in sys.modules:
            continue
        try:
            if importlib.util.find_spec(name) is not None:
                continue
        except (ImportError, ValueError, AttributeError):
            pass
        mod = _StubModule(name)
        mod.__path__ = []  # behaves as a package
        mod.__spec__ = importlib.machinery.ModuleSpec(name, loader=None, is_package=True)
        sys.modules[name] = mod
        parent, _, child = name.rpartition(".")
        if parent and parent in sys.modules:
            setattr(sys.modules[parent], child, mod)


def _patch_torch_private() -> None:
    try:
        import torch._inductor.codecache as cc

        if not hasattr(cc, "_reload_python_module_in_subproc"):
            cc._reload_python_module_in_subproc = lambda *a, **k: None
    except Exception:
        pass


def load():
    """Return the bare ``recpre`` package object with sub-modules importable as ``recpre.<name>``."""
    if not available():
        raise ImportError(f"reference not installed under {REF_ROOT}")
    if "recpre" in sys.modules and getattr(sys.modules["recpre"], "_b200_shim", False):
        return sys.modules["recpre"]
    _install_stubs()
    _patch_torch_private()
    pkg = types.ModuleType("recpre")
    pkg.__path__ = [os.path.join(REF_ROOT, "recpre")]
    pkg.__spec__ = importlib.machinery.ModuleSpec("recpre", loader=None, is_package=True)
    pkg._b200_shim = True
    sys.modules["recpre"] = pkg
    return pkg


def module(name: str):
    load()
    return importlib.import_module(f"recpre.{name}")


def build_train_model(model_name: str, gradient_checkpointing: bool = False, **overrides):
    """Construct the reference's training model through its own config factory."""
    cfgmod = module("config_dynamic")
    cfg = cfgmod.Config.from_name(model_name, **overrides)
    objective = {"op": None, "ignore_index": -100, "z_regularization": 0.0}
    return cfg.construct_model(objective=objective, gradient_checkpointing=gradient_checkpointing), cfg
