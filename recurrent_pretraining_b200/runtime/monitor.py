"""Observability: running means, step metrics, MFU against a peak table that knows the B200, optimizer telemetry,
and loggers (JSON lines always; wandb when installed and requested).

Counterpart of recpre/monitor.py:11-336 and train.py:545-662.  FLOPs are analytic (``ModelConfig.flops_per_token``)
instead of a meta-tensor trace; the peak table adds B200 entries (the reference's table raises on this GPU).
"""
from __future__ import annotations

import json
import math
import os
import time
from collections import deque

import torch

# dense bf16 peaks in FLOP/s by device-name substring (nominal; MFU is reported against these)
PEAK_FLOPS = {"B200": 2.25e15, "H200": 989e12, "H100": 989e12, "A100": 312e12, "MI250X": 191.5e12, "MI300X": 1307e12,
              "A6000": 155e12, "L40": 181e12, "4090": 165e12}


def peak_flops(device_name: str | None = None) -> float:
    if device_name is None:
        device_name = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
    for key, val in PEAK_FLOPS.items():
        if key.lower() in device_name.lower():
            return val
    return float("nan")


class RunningMean:
    def __init__(self, window: int = 32):
        self.buf = deque(maxlen=window)

    def update(self, v) -> None:
        self.buf.append(float(v))

    def compute(self) -> float:
        return sum(self.buf) / len(self.buf) if self.buf else float("nan")


class JsonlLogger:
    def __init__(self, path: str):
        os.makedirs(os.path.dirname(path), exist_ok=True)
        self.f = open(path, "a")

    def log_metrics(self, metrics: dict, step: int | None = None) -> None:
        rec = {k: (float(v) if torch.is_tensor(v) else v) for k, v in metrics.items()}
        rec["step"] = step
        self.f.write(json.dumps(rec, default=str) + "\n")
        self.f.flush()


def make_loggers(name: str, out_dir: str, run_name: str, project: str, rank: int) -> list:
    if rank != 0:
        return []
    loggers = [JsonlLogger(os.path.join(out_dir, "logs", f"{run_name}.jsonl"))]
    if name == "wandb":
        try:
            import wandb  # noqa: F401

            run = wandb.init(project=project, name=run_name, dir=out_dir, mode=os.environ.get("WANDB_MODE", "offline"))

            class _W:
                def log_metrics(self, metrics, step=None):
                    run.log({k: (float(v) if torch.is_tensor(v) else v) for k, v in metrics.items()}, step=step)

            loggers.append(_W())
        except Exception:
            pass
    return loggers


class StepTimer:
    """Wall-clock throughput between log points (device-synchronised only when read)."""

    def __init__(self):
        self.t0 = time.time()
        self.tokens = 0
        self.steps = 0
        self.flops = 0.0

    def add(self, tokens: int, flops: float) -> None:
        self.tokens += tokens
        self.steps += 1
        self.flops += flops

    def read_and_reset(self) -> dict:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dt = max(time.time() - self.t0, 1e-9)
        out = {"tokens_per_second": self.tokens / dt, "steps_per_second": self.steps / dt,
               "tflops": self.flops / dt / 1e12, "mfu": self.flops / dt / peak_flops()}
        self.__init__()
        return out


@torch.no_grad()
def optimizer_telemetry(model, optimizer) -> dict:
    """Gradient / parameter norms of selected layers (recpre/monitor.py:39-137): q-projection and second FFN matrix
    gradient norms per block, global L1/L2 parameter norms."""
    out, l1, l2 = {}, 0.0, 0.0
    for name, p in model.named_parameters():
        pf = p.detach().float()
        l1 += pf.abs().sum().item()
        l2 += pf.pow(2).sum().item()
        if p.grad is None:
            continue
        if name.endswith("attn.Wqkv.weight"):
            E = p.shape[1]
            out[f"grad_norm_q/{name}"] = p.grad[:E].float().norm().item()
        elif name.endswith("mlp.proj.weight"):
            out[f"grad_norm_ffn2/{name}"] = p.grad.float().norm().item()
    out["param_l1"], out["param_l2"] = l1, math.sqrt(l2)
    return out


def enable_monitoring(model, on: bool = True) -> None:
    for m in model.modules():
        if hasattr(m, "monitoring"):
            m.monitoring = on


def harvest_metrics(model) -> dict:
    out = {}
    for m in model.modules():
        lm = getattr(m, "latest_metrics", None)
        if lm:
            out.update(lm)
    return out
