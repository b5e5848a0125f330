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


def peak_flops(device_name: str | None = None, precision: str = "bf16") -> float:
    """Nominal dense tensor peak of the device for the run's precision string (``"bf16-mixed"``, ``"32-true"``, ...):
    halved for fp32, quartered for fp64, doubled for 8-bit, as in recpre/monitor.py:195-245 -- but with entries for the
    GPUs that table does not know (it raises on a B200)."""
    if device_name is None:
        device_name = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
    mult = 0.5 if "32" in precision else 0.25 if "64" in precision else 2.0 if "8" in precision else 1.0
    for key, val in PEAK_FLOPS.items():
        if key.lower() in device_name.lower():
            return val * mult
    return float("nan")


def num_params(model, only_trainable: bool = False) -> int:
    return sum(p.numel() for p in model.parameters() if p.requires_grad or not only_trainable)


def estimate_flops_per_token(n_params: int, cfg) -> int:
    """The reference's closed-form estimate (recpre/monitor.py:152-160): ``3 * (6 P + 12 L H Q T)``."""
    heads = getattr(cfg, "n_heads", None) or cfg.num_attention_heads
    return 3 * (6 * n_params + 12 * cfg.n_layer * heads * cfg.head_size * cfg.block_size)


def measure_flops(cfg, micro_batch_size: int = 1, gradient_checkpointing: bool = False) -> float:
    """FLOPs of one forward + backward pass over ``micro_batch_size`` sequences of ``block_size`` tokens, counted by
    torch's FLOP counter on a meta-device copy of the model (the measurement behind the reference's MFU,
    recpre/monitor.py:163-192).  Falls back to the analytic count when the model cannot run on meta tensors."""
    import copy

    from torch.utils.flop_counter import FlopCounterMode

    try:
        with torch.device("meta"):
            meta = copy.deepcopy(cfg).construct_model(gradient_checkpointing=gradient_checkpointing)
            x = torch.randint(0, cfg.padded_vocab_size, (micro_batch_size, cfg.block_size))
            counter = FlopCounterMode(display=False)
            with counter:
                meta(x, labels=x)["loss"].backward()
        depths = getattr(meta, "last_depths", None)
        return float(counter.get_total_flops()), depths
    except Exception:  # noqa: BLE001  (any op without a meta kernel)
        n, k = (cfg.mean_recurrence - cfg.mean_backprop_depth, cfg.mean_backprop_depth) if cfg.is_recurrent else (0, 0)
        return cfg.flops_per_token(cfg.block_size, n, k, gradient_checkpointing) * cfg.block_size * micro_batch_size, (n, k)


_mfu_cache: dict = {}


def mfu_metrics(tokens_per_second: float, world_size: int, model, precision: str = "bf16-mixed",
                measure: bool = True, device_name: str | None = None):
    """(FLOPs per token, achieved TFLOP/s of the whole job, MFU per device) -- the triple of the reference's
    ``get_MFU_metrics`` (recpre/monitor.py:248-266); model constants are cached per model object."""
    c = _mfu_cache.get(id(model))
    if c is None:
        n = num_params(model)
        cfg = model.config
        if measure:
            total, _ = measure_flops(cfg, 1, getattr(model, "gradient_checkpointing", False))
            per_token = total / cfg.block_size
        else:
            per_token = estimate_flops_per_token(n, cfg)
        c = _mfu_cache[id(model)] = {"num_params": n, "num_flop_per_token": per_token,
                                     "peak_flops": peak_flops(device_name, precision)}
    flops = c["num_flop_per_token"] * tokens_per_second
    return c["num_flop_per_token"], flops / 1e12, flops / world_size / c["peak_flops"]


def measure_peak_flops(sizes=(2048, 4096, 8192), batch: int = 8, runs: int = 20) -> list:
    """Achieved dense bf16 matmul rate of this GPU: the library's batched GEMM and the in-tree tcgen05 GEMM on square
    problems, timed with CUDA events (the counterpart of recpre/monitor.py:269-336, which compares against an A100 peak).
    ``python -m recurrent_pretraining_b200.runtime.monitor`` prints the table."""
    from ..ops import cuda as C

    nominal = peak_flops()
    rows = []
    for n in sizes:
        a = torch.randn(batch, n, n, device="cuda").bfloat16()
        b = torch.randn(batch, n, n, device="cuda").bfloat16()

        def timed(fn):
            fn()
            torch.cuda.synchronize()
            ts = []
            for _ in range(runs):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) / 1e3)
            ts.sort()
            return ts[len(ts) // 2]

        t_lib = timed(lambda: torch.bmm(a, b))
        t_own = timed(lambda: [C.gemm(a[i], b[i], b_mn=True) for i in range(batch)])
        fl = 2.0 * n ** 3 * batch
        rows.append({"n": n, "batch": batch, "library_tflops": fl / t_lib / 1e12, "tcgen05_tflops": fl / t_own / 1e12,
                     "library_frac_of_nominal": fl / t_lib / nominal, "tcgen05_frac_of_nominal": fl / t_own / nominal})
        print(rows[-1], flush=True)
    return rows


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


def adam_effective_lr(grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-element ratio of the Adam direction to the raw gradient, ``m / (sqrt(v) + eps) / g`` (``/ eps`` where the
    gradient is below eps): how much the optimizer amplifies or damps each coordinate, without bias correction and
    without the scheduled learning rate (recpre/monitor.py:24-36)."""
    g = grad.float()
    direction = exp_avg.float() / (exp_avg_sq.float().sqrt() + eps)
    return torch.where(g.abs() > eps, direction / g, direction / eps)


def _moments(optimizer, p):
    """(exp_avg, exp_avg_sq, eps) of one parameter for torch-style optimizers and for the flat fused optimizer (full-size
    state only; sharded state holds pieces and is skipped)."""
    st = getattr(optimizer, "state", None)
    if isinstance(st, dict) or hasattr(st, "get"):
        ps = st.get(p) if hasattr(st, "get") else None
        if ps and "exp_avg" in ps and "exp_avg_sq" in ps:
            eps = next((g["eps"] for g in optimizer.param_groups if any(q is p for q in g["params"])), 1e-8)
            return ps["exp_avg"], ps["exp_avg_sq"], eps
    groups = getattr(optimizer, "groups", None)
    if groups is not None and getattr(optimizer, "plans", None) is None:
        if hasattr(optimizer, "finish_deferred"):
            optimizer.finish_deferred()
        for g, h in zip(groups, optimizer.param_groups):
            for q, off in zip(g.params, g.offsets):
                if q is p:
                    n = p.numel()
                    return (g.state["m"][off:off + n].view(p.shape), g.state["v"][off:off + n].view(p.shape),
                            h["eps"])
    return None


@torch.no_grad()
def optimizer_telemetry(model, optimizer) -> dict:
    """Optimizer-side telemetry of one step (recpre/monitor.py:39-137, same metric names): query / second-FFN gradient
    norms per layer, RMS of ``g^2 / v`` per parameter (mean over parameters, and for the embedding), effective Adam
    learning rates of the q / k / v rows and of the second FFN matrix, mean local L1 gradient norm, and parameter norms
    (all, core block, embedding, everything but the embedding)."""
    cfg = getattr(model, "config", None)
    E = getattr(cfg, "n_embd", None)
    kv = getattr(cfg, "head_size", 0) * getattr(cfg, "n_query_groups", 0) if cfg is not None else 0
    wte = getattr(getattr(model, "transformer", None), "wte", None)
    out: dict = {}
    qkv_i = ffn_i = 0
    rms_sum, rms_n, l1_grads = 0.0, 0, []
    sq_all = sq_core = sq_wte = sq_rest = 0.0
    l1_params = []
    for name, p in model.named_parameters():
        pf = p.detach().float()
        sq = pf.pow(2).sum().item()
        sq_all += sq
        l1_params.append(pf.abs().sum().item())
        if ".core_block." in name:
            sq_core += sq
        if ".wte." in name:
            sq_wte += sq
        else:
            sq_rest += sq
        g = p.grad
        if g is None:
            continue
        is_qkv = "qkv" in name.lower() and name.endswith("weight")
        is_ffn2 = ".mlp." in name and "proj" in name and name.endswith("weight")
        finite = bool(torch.isfinite(g).all())
        if is_qkv:
            if not finite:
                out[f"query_grad_{qkv_i}"] = float("nan")
            elif E and g.dim() == 2 and g.shape[1] == E:
                out[f"query_grad_{qkv_i}"] = g[:E].float().norm().item()
        if is_ffn2:
            out[f"ffn2_grad_{ffn_i}"] = g.float().norm().item() if finite else float("nan")
        if finite:
            l1_grads.append(g.float().abs().sum().item())
            mom = _moments(optimizer, p)
            if mom is not None and mom[1].shape == g.shape:
                m, v, eps = mom
                rms = (g.float().pow(2) / v.float().clamp(min=eps ** 2)).mean().sqrt().item()
                rms_sum += rms
                rms_n += 1
                if wte is not None and p is wte.weight:
                    out["embed_RMS"] = rms
                if is_qkv and E and g.dim() == 2 and g.shape[1] == E:
                    lr = adam_effective_lr(g, m, v, eps)
                    out[f"q_effective_lr_{qkv_i}"] = lr[:E].mean().item()
                    out[f"k_effective_lr_{qkv_i}"] = lr[E:E + kv].mean().item()
                    out[f"v_effective_lr_{qkv_i}"] = lr[E + kv:].mean().item()
                if is_ffn2:
                    out[f"ffn2_effective_lr_{ffn_i}"] = adam_effective_lr(g, m, v, eps).mean().item()
        qkv_i += int(is_qkv)
        ffn_i += int(is_ffn2)
    if rms_n:
        out["avg_RMS"] = rms_sum / rms_n
    if l1_grads:
        out["local_l1_grad_norm"] = sum(l1_grads) / len(l1_grads)
    out["l2_param_norm"] = math.sqrt(sq_all)
    out["l1_param_norm"] = sum(l1_params) / max(len(l1_params), 1)
    out["core_block_l2_param_norm"] = math.sqrt(sq_core)
    out["word_embed_l2_param_norm"] = math.sqrt(sq_wte)
    out["model_l2_param_norm"] = math.sqrt(sq_rest)
    return out


def enable_monitoring(model, on: bool = True) -> None:
    for m in model.modules():
        if hasattr(m, "monitoring"):
            m.monitoring = on


def harvest_metrics(model, metrics: dict | None = None) -> dict:
    """Collect (and clear) the ``latest_metrics`` of every module; one-element tensors become numbers.  With a
    ``metrics`` dict the values are merged into it, as ``disable_monitoring_and_retrieve_metrics(module, metrics)`` of
    the reference does (recpre/monitor.py:16-21)."""
    out = {} if metrics is None else metrics
    for m in model.modules():
        lm = getattr(m, "latest_metrics", None)
        if lm:
            out.update({k: (v.item() if torch.is_tensor(v) and v.numel() == 1 else v) for k, v in lm.items()})
            m.latest_metrics = {}
    return out


if __name__ == "__main__":
    measure_peak_flops()
