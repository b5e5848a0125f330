"""Optimizers: parameter grouping, the fused flat-buffer AdamW, and the named research optimizers."""
from .groups import get_param_groups  # noqa: F401
from .registry import get_optimizer  # noqa: F401
