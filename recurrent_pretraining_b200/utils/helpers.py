"""Small helpers that scripts written against the reference expect to find (recpre/utils.py:53-110,338-350,489-637,
730-866,1363-1397,1520-1567,1629-1720): rounding and counting, checkpoint-directory conventions, hyper-parameter
capture, label remapping for restricted-vocabulary evaluation, a cycling iterator, a closed-form parameter count,
abacus parameter groups, and the linear + cross-entropy head module.  Restated here without lightning / jsonargparse.
"""
from __future__ import annotations

import dataclasses
import inspect
import json
import math
import shutil
from pathlib import Path
from typing import Any, Iterable, Mapping, Optional, Sequence

import torch
import torch.nn as nn


def find_multiple(n: int, k: int) -> int:
    """Smallest multiple of k that is not below n."""
    assert k > 0
    return n if n % k == 0 else n + k - (n % k)


def num_parameters(module: nn.Module, requires_grad: Optional[bool] = None) -> int:
    """Parameter count; ``requires_grad`` True / False restricts to trainable / frozen parameters."""
    return sum(p.numel() for p in module.parameters() if requires_grad is None or p.requires_grad == requires_grad)


def reset_parameters(module: nn.Module) -> None:
    """Call ``reset_parameters`` on every submodule that has one."""
    for m in module.modules():
        fn = getattr(m, "reset_parameters", None)
        if callable(fn) and m is not module:
            fn()


def check_valid_checkpoint_dir(checkpoint_dir: Path, model_filename: str = "lit_model.pth") -> None:
    """Raise SystemExit with a readable message unless the directory holds a model file, its config and a tokenizer."""
    checkpoint_dir = Path(checkpoint_dir)
    needed = {model_filename: (checkpoint_dir / model_filename).is_file(),
              "model_config.yaml": (checkpoint_dir / "model_config.yaml").is_file(),
              "tokenizer.json OR tokenizer.model": (checkpoint_dir / "tokenizer.json").is_file()
              or (checkpoint_dir / "tokenizer.model").is_file(),
              "tokenizer_config.json": (checkpoint_dir / "tokenizer_config.json").is_file()}
    if checkpoint_dir.is_dir() and all(needed.values()):
        return
    missing = [k for k, ok in needed.items() if not ok]
    others = sorted(str(p.parent) for p in Path("checkpoints").glob("*/*/") if p.is_dir()) if Path("checkpoints").is_dir() \
        else []
    hint = ("\nCheckpoint directories found:\n" + "\n".join(f"  --checkpoint_dir '{o}'" for o in others)) if others else ""
    raise SystemExit(f"--checkpoint_dir {str(checkpoint_dir.absolute())!r} is missing: {missing}.{hint}")


def extend_checkpoint_dir(checkpoint_dir: Path) -> Path:
    """``org/model`` -> ``checkpoints/org/model`` when only the latter exists (relative paths only)."""
    checkpoint_dir = Path(checkpoint_dir)
    candidate = Path("checkpoints") / checkpoint_dir
    use = (not checkpoint_dir.is_dir() and not checkpoint_dir.is_absolute()
           and (not checkpoint_dir.parts or checkpoint_dir.parts[0] != "checkpoints") and candidate.exists())
    return candidate if use else checkpoint_dir


def copy_config_files(source_dir: Path, out_dir: Path) -> None:
    """Copy the generation / model configs and the tokenizer files that exist in ``source_dir``."""
    for name in ("generation_config.json", "model_config.yaml", "tokenizer.json", "tokenizer.model",
                 "tokenizer_config.json"):
        src = Path(source_dir) / name
        if src.exists():
            shutil.copy(src, out_dir)


def flatten_dict(d: Mapping, parentkey: str = "", sep: str = "_", coerce_to_str: bool = False) -> dict:
    """Nested mapping -> flat dict with joined keys (for loggers that want scalars)."""
    out: dict = {}
    for k, v in d.items():
        key = f"{parentkey}{sep}{k}" if parentkey else str(k)
        if isinstance(v, Mapping) and v:
            out.update(flatten_dict(v, key, sep, coerce_to_str))
        else:
            out[key] = str(v) if coerce_to_str else v
    return out


def capture_hparams() -> dict:
    """The caller's local variables as a plain dict: scalars and paths as they are, dataclasses as dicts, the rest as
    strings."""
    frame = inspect.currentframe().f_back
    out = {}
    for name, value in frame.f_locals.items():
        if value is None or isinstance(value, (int, float, str, bool, Path)):
            out[name] = value
        elif dataclasses.is_dataclass(value) and not isinstance(value, type):
            out[name] = dataclasses.asdict(value)
        else:
            out[name] = str(value)
    return out


def save_hyperparameters(settings, checkpoint_dir: Path) -> None:
    """Write the run's settings (a dataclass or a dict) to ``hyperparameters.yaml`` beside the checkpoint."""
    import yaml

    data = dataclasses.asdict(settings) if dataclasses.is_dataclass(settings) else dict(settings)
    Path(checkpoint_dir).mkdir(parents=True, exist_ok=True)
    with open(Path(checkpoint_dir) / "hyperparameters.yaml", "w", encoding="utf-8") as f:
        yaml.safe_dump(json.loads(json.dumps(data, default=str)), f)


def save_config(config, checkpoint_dir: Path) -> None:
    """Write the model config to ``model_config.yaml``."""
    import yaml

    data = config.to_dict() if hasattr(config, "to_dict") else dataclasses.asdict(config)
    Path(checkpoint_dir).mkdir(parents=True, exist_ok=True)
    with open(Path(checkpoint_dir) / "model_config.yaml", "w", encoding="utf-8") as f:
        yaml.safe_dump(json.loads(json.dumps(data, default=str)), f)


def parse_devices(devices) -> int:
    if devices in (-1, "auto"):
        return torch.cuda.device_count() or 1
    if isinstance(devices, int) and not isinstance(devices, bool) and devices > 0:
        return devices
    raise ValueError(f"Devices must be 'auto' or a positive integer, got: {devices!r}")


def get_default_supported_precision(training: bool) -> str:
    """``bf16-mixed`` / ``bf16-true`` where bf16 exists, else the fp16 forms."""
    no_bf16 = torch.cuda.is_available() and not torch.cuda.is_bf16_supported()
    kind = "mixed" if training else "true"
    return f"16-{kind}" if no_bf16 else f"bf16-{kind}"


def map_old_state_dict_weights(state_dict: dict, mapping: Mapping, prefix: str) -> dict:
    """Rename ``prefix + old`` to ``prefix + new`` for every pair of ``mapping`` present in the state dict."""
    for old, new in mapping.items():
        if prefix + old in state_dict:
            state_dict[prefix + new] = state_dict.pop(prefix + old)
    return state_dict


def slice_logits_remap_labels(logits: torch.Tensor, targets: torch.Tensor, target_range: Sequence[int],
                              ignore_indices: Sequence[int] = (-1,)) -> tuple[torch.Tensor, torch.Tensor]:
    """Restrict a classification to the (sorted, not necessarily contiguous) vocabulary ids in ``target_range``: the
    logits keep only those columns, and targets equal to the i-th id become i (other targets are left alone: they are
    expected to be ignore values)."""
    ids = list(target_range)
    assert ids and min(ids) >= 0 and max(ids) < logits.size(-1) and sorted(ids) == ids
    out = targets.clone()
    for new, old in enumerate(ids):
        out[targets == old] = new
    return logits[..., ids], out


class CycleIterator:
    """Cycle through an iterable for ever, re-creating its iterator at every pass (nothing is cached) and counting the
    passes in ``epoch``."""

    def __init__(self, iterable: Iterable) -> None:
        self.iterable, self.epoch, self._it = iterable, 0, None

    def __iter__(self):
        return self

    def __next__(self) -> Any:
        if self._it is None:
            self._it = iter(self.iterable)
        try:
            return next(self._it)
        except StopIteration:
            self._it = iter(self.iterable)
            self.epoch += 1
            return next(self._it)


def param_count_estimator(width: int, depth: int, vocab_size: int, n_head: int, head_size: int, n_query_groups: int,
                          intermediate_size: int) -> int:
    """Closed-form parameter count of a gated-MLP transformer with untied embedding and head and two norms per block."""
    attn = width * (n_head + 2 * n_query_groups) * head_size + head_size * n_head * width
    mlp = 3 * width * intermediate_size
    return depth * (attn + mlp + 2 * width) + vocab_size * width + width + width * vocab_size


def get_abacus_param_groups(named_parameters, lr: float, no_weight_decay_for_bias_and_norm_params: bool = True,
                            increase_abacus_lr_multiplier: float = 0.0) -> list:
    """Parameter groups with an own (multiplied) learning rate for the abacus position embedding."""
    decay, no_decay, abacus = [], [], None
    boost = increase_abacus_lr_multiplier > 0.0
    for name, p in named_parameters:
        low = name.lower()
        if boost and "abacus" in low:
            abacus = p
        elif no_weight_decay_for_bias_and_norm_params and ("norm" in low or "bias" in low):
            no_decay.append(p)
        else:
            decay.append(p)
    groups = []
    if decay:
        groups.append({"params": decay, "lr": lr})
    if no_decay:
        groups.append({"params": no_decay, "lr": lr, "weight_decay": 0.0})
    if boost:
        assert abacus is not None, "no abacus parameter found, but a learning-rate multiplier was given for it"
        groups.append({"params": [abacus], "lr": lr * increase_abacus_lr_multiplier,
                       "increase_abacus_lr_multiplier": increase_abacus_lr_multiplier})
    return groups


class LinearCrossEntropyLoss(nn.Linear):
    """A bias-free output projection that returns the loss when given labels: ``forward(x)`` -> logits,
    ``forward(x, y)`` -> mean cross entropy without keeping the logits (on CUDA the head GEMM's epilogue produces the
    softmax partials, ``ops.linear_cross_entropy``; on CPU rows are processed in chunks).  Stays an ``nn.Linear`` so
    that code which looks for linear layers (init, parameter groups) finds it."""

    def __init__(self, in_features: int, out_features: int, device=None, dtype=None, ignore_index: int = -100,
                 chunk_size: int = 1024, init_method=None):
        self.init_method = None
        super().__init__(in_features, out_features, bias=False, device=device, dtype=dtype)
        self.ignore_index, self.chunk_size, self.init_method = ignore_index, chunk_size, init_method
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if self.init_method is not None:
            self.init_method(self.weight)
        else:
            std = math.sqrt(1 / self.in_features)
            nn.init.trunc_normal_(self.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)

    def forward(self, x: torch.Tensor, y: Optional[torch.Tensor] = None) -> torch.Tensor:
        if y is None:
            return torch.matmul(x, self.weight.t())
        from ..ops import functional as ops

        return ops.linear_cross_entropy(x.reshape(-1, self.in_features), self.weight, y.reshape(-1), 1.0,
                                        self.ignore_index, 0.0)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias=False"
