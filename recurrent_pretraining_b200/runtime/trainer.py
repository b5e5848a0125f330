"""Pretraining driver: start-up, hot loop, validation at several recurrence depths, logging, checkpointing and the
failure guards of the reference (train.py:183-537, 865-1076).

Behaviour kept from the reference: resume from the newest checkpoint of the run name; warm-up collectives that fail
early; non-finite loss raises the exit flag; the exit flag is MIN-reduced over ranks every 32 micro-steps (training
stops only when every rank asked for it); optional checkpoint N minutes before the SLURM wall-time; the process group
is always destroyed on exit.
"""
from __future__ import annotations

import functools
import math
import os
import subprocess
import time
from typing import Optional

import torch
import torch.distributed as dist

from ..data import (BufferShuffledParquet, DataScheduler, DataSchedulerTracker, ParquetStream, RandomTokens, StatefulLoader, TextRows,
                    Tokenizer, WeightedMixture, apply_tld, generic_collate_fn)
from ..optim.schedules import get_batch_size, get_lr
from ..parallel.fabric import Fabric
from . import checkpoint as ckpt
from .engine import TrainEngine
from .monitor import (RunningMean, StepTimer, enable_monitoring, harvest_metrics, make_loggers, optimizer_telemetry)


def device_health_check() -> None:
    """Query the device manager before CUDA initialisation; a GPU that cannot be queried is a node failure
    (train.py:25-28).  Read-only NVML calls."""
    try:
        import pynvml

        pynvml.nvmlInit()
        for i in range(pynvml.nvmlDeviceGetCount()):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            pynvml.nvmlDeviceGetMemoryInfo(h)
    except ImportError:
        return
    except Exception as exc:  # noqa: BLE001
        if os.environ.get("B200_SKIP_HEALTH_CHECK") != "1" and torch.cuda.is_available():
            raise RuntimeError(f"Node failure! device manager error: {exc}") from exc


def set_torch_flags(cfg) -> None:
    torch.set_float32_matmul_precision(cfg.matmul_precision)
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True


def setup_fabric(cfg) -> Fabric:
    """``fabric_strategy`` names of the reference (train.py:111-158) mapped onto the gradient-sync modes of
    ``parallel.fabric``: the DDP names run the overlapped reduce-scatter + sharded update (``p2p``); ``zero`` and
    ``fsdp-grad`` the same (gradients and optimizer state are what they shard); ``fsdp-full`` / ``fsdp-hybrid*`` / ``zero3``
    additionally shard the fp32 parameters and gather the bf16 weights in the forward pass (``zero3``)."""
    sync = cfg.grad_sync
    strategy = cfg.fabric_strategy
    if strategy in ("fsdp-full", "fsdp-hybrid", "fsdp-hybrid2", "zero3"):
        if sync not in (None, "zero3"):
            raise ValueError(f"fabric_strategy {strategy!r} shards parameters: grad_sync must be zero3 (or unset)")
        sync = "zero3" if torch.cuda.is_available() else "flat"
    elif strategy.startswith("fsdp"):
        if sync not in (None, "p2p"):
            raise ValueError(f"fabric_strategy {strategy!r} runs on the fused sharded path (grad_sync: p2p)")
        sync = "p2p" if torch.cuda.is_available() else "flat"
    elif strategy not in ("simple-ddp", "ddp", "single", "zero"):
        raise ValueError(f"fabric_strategy {strategy!r}: tensor parallelism through AxoNN is an external library in the "
                         "reference and is not provided; use simple-ddp, zero, zero3 or fsdp-*")
    if sync is None and torch.cuda.is_available() and int(os.environ.get("WORLD_SIZE", os.environ.get("SLURM_NTASKS", 1))) > 1:
        sync = "p2p"
    return Fabric.from_env(grad_sync=sync, precision=cfg.fabric_precision)


# ------------------------------------------------------------------------------------------------------
def _make_source(entry, cfg, fabric, split_dir: str, seed: int):
    vocab, block = cfg.model_config.padded_vocab_size, cfg.loader_block_size
    if entry.type == "rngds":
        return RandomTokens(vocab, block, seed=seed, process_rank=fabric.global_rank)
    folder = entry.data_dir or split_dir
    if entry.type == "pqds":
        return BufferShuffledParquet(folder, seed=seed, shuffle=cfg.shuffle_blocks, num_processes=fabric.world_size,
                                     process_rank=fabric.global_rank, prefix=entry.prefix,
                                     shuffle_filenames=cfg.shuffle_filenames, return_data_id=entry.return_data_id,
                                     data_id=entry.prefix)
    if entry.type == "pqds-pure":
        return ParquetStream(folder, seed=seed, shuffle=cfg.shuffle_blocks, num_processes=fabric.world_size,
                             process_rank=fabric.global_rank, prefix=entry.prefix,
                             shuffle_filenames=cfg.shuffle_filenames, return_data_id=entry.return_data_id,
                             data_id=entry.prefix)
    if entry.type == "hfds":
        sig = entry.data_signature or cfg.data_signature
        return TextRows(os.path.join(folder, entry.prefix), sig, fabric.world_size, fabric.global_rank,
                        shuffle=cfg.shuffle_blocks, seed=seed, data_id=entry.prefix,
                        repetitions=getattr(entry, "repetitions", None), return_data_id=entry.return_data_id)
    raise ValueError(f"Unsupported dataset type {entry.type}")


def create_dataloader(cfg, fabric, tokenizer, entries, split_dir, seed, scheduler=None, prefetch=4):
    sources = [_make_source(e, cfg, fabric, split_dir, seed + i) for i, e in enumerate(entries)]
    ds = sources[0] if len(sources) == 1 else WeightedMixture(sources, [e.weight for e in entries], seed, scheduler)
    all_tensors = cfg.all_block_size_tensors or all(e.type in ("rngds", "pqds", "pqds-pure") for e in entries)
    collate = functools.partial(generic_collate_fn, tokenizer=tokenizer, block_size=cfg.loader_block_size,
                                pad_to_block_size=cfg.pad_to_block_size, add_bos=cfg.add_bos, add_eos=cfg.add_eos,
                                collate_checks_enabled=cfg.collate_checks_enabled,
                                all_block_size_tensors=all_tensors)
    return StatefulLoader(ds, cfg.micro_batch_size, collate, prefetch=prefetch)


def derive_precision(precision: str, all_reduce_dtype: Optional[str] = None) -> dict:
    """Dtypes that a precision string stands for (train.py:802-822 of the reference builds torch-FSDP's MixedPrecision
    from the same rule): compute copy of the parameters, gradient reduction, buffers."""
    param = torch.bfloat16 if "bf16" in precision else torch.float16 if "16" in precision else torch.float32
    reduce = torch.float32 if "mixed" in precision else param
    if all_reduce_dtype is not None:
        reduce = torch.float16 if all_reduce_dtype in ("16", "fp16", "fp16-mixed") else \
            torch.bfloat16 if all_reduce_dtype in ("bf16", "bf16-mixed") else torch.float32
    return {"param_dtype": param, "reduce_dtype": reduce, "buffer_dtype": torch.float32}


def get_attention_mask(input_ids, tokenizer=None, cache_attn: bool = True, doc_block_attn: bool = True):
    """Pretraining packs documents without a block mask and without explicit positions: (mask, position_ids) =
    (None, None), as in the reference (train.py:825-827); the models then run plain causal attention."""
    return None, None


def warmup_or_early_fail_allreduce(fabric) -> None:
    """Growing all-reduces so that a broken fabric fails before any real work (train.py:965-982)."""
    if not fabric.is_distributed:
        return
    for mb in (16, 32, 64, 128):
        t = torch.ones(mb * 2**20 // 4, device=fabric.device)
        dist.all_reduce(t)
        if not bool((t[:4] == fabric.world_size).all()):
            raise RuntimeError("all-reduce warm-up produced a wrong sum")
    fabric.barrier()


def slurm_seconds_left() -> Optional[float]:
    job = os.environ.get("SLURM_JOB_ID")
    if not job:
        return None
    try:
        out = subprocess.run(["squeue", "-h", "-j", job, "-o", "%L"], capture_output=True, text=True, timeout=10).stdout
        parts = out.strip().replace("-", ":").split(":")
        nums = [int(p) for p in parts]
        mult = [1, 60, 3600, 86400]
        return float(sum(n * m for n, m in zip(reversed(nums), mult)))
    except Exception:
        return None


_ELLIS_FUSED = {"update_clipping", "atan_adam", "running_init", "decouple_wd"}
_ELLIS_OFF = {"nesterov": False, "eps_adjustment": False, "kahan_sum_compensation": False, "buffer_dtype": None,
              "tensor_wise_finite_check": False, "tensor_wise_gradient_normalization": False,
              "adafactor_like_beta_corrections": False, "brute_force_clip": None, "poly_ema_p": None, "foreach": None}


def fused_optimizer_flags(name: str, optim_config: dict) -> Optional[dict]:
    """Keyword flags for ``TrainEngine`` when the optimizer can run on the fused flat path, else None.  Covered: AdamW,
    and ELLISAdam with any of update_clipping / atan_adam / running_init / decouple_wd (the flags of the reference's
    production run, launch_configs/frontier_nebel_512_nodes.yaml:28-41); every other ELLISAdam option must be off."""
    if name in ("AdamW", "FusedAdamW"):
        return {}
    if name != "ELLISAdam":
        return None
    for k, off in _ELLIS_OFF.items():
        if optim_config.get(k, off) not in (off, False, None):
            return None
    return {"atan2": bool(optim_config.get("atan_adam", False)),
            "update_clipping": bool(optim_config.get("update_clipping", False)),
            "running_init": bool(optim_config.get("running_init", False)),
            "decouple_wd": bool(optim_config.get("decouple_wd", True))}


# ------------------------------------------------------------------------------------------------------
def startup(cfg, fabric: Fabric) -> dict:
    t0 = time.time()
    if fabric.global_rank == 0:
        os.makedirs(cfg.out_dir, exist_ok=True)
        cfg.dump(os.path.join(cfg.out_dir, "run_config.json"))
        import json

        with open(os.path.join(cfg.out_dir, "model_config.json"), "w") as f:
            json.dump(cfg.model_config.to_dict(), f, indent=2, default=str)
    tokenizer = Tokenizer(cfg.tokenizer_path or None)
    fabric.seed_everything(cfg.seed)
    mc = cfg.model_config
    if cfg.block_size != mc.block_size and not cfg.ignore_block_size_mismatch:
        mc.block_size = cfg.block_size
    # as in the reference (train.py:248-253) the objective names the tokenizer's pad id; the training loss ignores only
    # -100 (recpre/model_dynamic.py:1133-1134), the validation loss skips the pad id as well
    objective = {"ignore_index": tokenizer.pad_id if tokenizer.pad_id is not None else -1,
                 "z_regularization": cfg.z_regularization, "label_smoothing": cfg.label_smoothing}
    with torch.device(fabric.device):
        model = mc.construct_model(objective=objective, gradient_checkpointing=cfg.gradient_checkpointing)
    if cfg.model_checkpoint:
        sd = torch.load(cfg.model_checkpoint, map_location="cpu", weights_only=False)
        sd = ckpt.strip_wrapper_prefixes(sd.get("model", sd))
        model.load_state_dict(sd, strict=False)
    oc = dict(cfg.optim_config)
    lr = oc.pop("lr", 4e-4)
    max_steps = cfg.max_steps
    lr_fn = functools.partial(get_lr, lr, warmup_steps=cfg.warmup_steps, max_steps=max_steps,
                              cooldown_steps=cfg.cooldown_steps, schedule=cfg.lr_schedule, min_lr=cfg.min_lr)
    optimizer = None
    fused_flags = fused_optimizer_flags(cfg.optimizer, oc) if fabric.device.type == "cuda" else None
    use_fused = fused_flags is not None
    if not use_fused:
        from ..optim import get_optimizer, get_param_groups

        model.to(fabric.device)
        groups = get_param_groups(model.named_parameters(), cfg.no_weight_decay_for_bias_and_norm_params)
        optimizer = get_optimizer(cfg.optimizer, model=model, use_zero=cfg.fabric.optim_sharding)(groups, lr=lr, **oc)
    ellis = cfg.optimizer == "ELLISAdam"      # its constructor defaults differ from AdamW's (recpre/optim.py:729-735)
    engine = TrainEngine(model, fabric, lr=lr, weight_decay=oc.get("weight_decay", 1e-2 if ellis else 0.1),
                         betas=oc.get("betas", (0.9, 0.99) if ellis else (0.9, 0.95)),
                         eps=oc.get("eps", 1e-6 if ellis else 1e-8), grad_clip=cfg.grad_clip,
                         grad_accum=cfg.gradient_accumulation_steps, skip_first_step=cfg.skip_first_optimizer_step,
                         no_weight_decay_for_bias_and_norm_params=cfg.no_weight_decay_for_bias_and_norm_params,
                         optimizer=optimizer, lr_fn=lambda step: lr_fn(step=step), **(fused_flags or {}))
    tracker = DataSchedulerTracker([e.weight for e in cfg.data_config["train_data"]])
    scheduler = DataScheduler(tracker, cfg.data_config["train_data"], max_steps)
    train_loader = create_dataloader(cfg, fabric, tokenizer, cfg.data_config["train_data"], cfg.train_data_dir,
                                     cfg.seed, scheduler)
    val_loader = create_dataloader(cfg, fabric, tokenizer, cfg.data_config.get("val_data") or
                                   cfg.data_config["train_data"], cfg.val_data_dir or cfg.train_data_dir,
                                   cfg.seed + 10_000, prefetch=0)
    state = {"model": model, "engine": engine, "train_dataloader": train_loader, "val_dataloader": val_loader,
             "data_scheduler": scheduler, "tokenizer": tokenizer, "microbatch_step": 0, "optimizer_step": 0,
             "is_accumulating": False, "metrics": {}, "should_exit_training": False,
             "model_config": mc.to_dict()}
    if cfg.resume:
        path = ckpt.find_latest(cfg.out_dir, cfg.run_name, fabric.local_rank)
        if path is not None:
            ckpt.load_checkpoint(fabric, state, path, strict=False)
            engine.micro_step = state["microbatch_step"]
            engine.window_base = engine.micro_step
            engine.optimizer_step = state["optimizer_step"]
            fabric.print(f"Resumed from {path} at micro-batch step {state['microbatch_step']}")
    fabric.barrier()
    path = "fused flat-buffer kernels" if engine.mode == "fused" else "torch optimizer on unflattened parameters"
    fabric.print(f"optimizer {cfg.optimizer} runs on the {path}; gradient sync: {fabric.grad_sync}")
    fabric.print(f"start-up took {time.time() - t0:.1f}s; {sum(p.numel() for p in model.parameters()):,} parameters")
    return state


@torch.no_grad()
def validate(cfg, fabric, state) -> dict:
    """Loss at each depth in ``partial_depth_eval + [mean_recurrence]`` over ``eval_iters`` batches, averaged over
    ranks (train.py:343-386)."""
    model, mc = state["model"], cfg.model_config
    depths = list(cfg.partial_depth_eval) + [mc.mean_recurrence] if mc.is_recurrent else [0]
    fabric.sync_parameters()
    model.eval()
    sums = torch.zeros(len(depths), device=fabric.device)
    n = 0
    ignore = (getattr(model, "objective", None) or {}).get("ignore_index", -100)
    for i, (x, y, _) in enumerate(state["val_dataloader"]):
        if i >= cfg.eval_iters:
            break
        x, y = x.to(fabric.device, non_blocking=True), y.to(fabric.device, non_blocking=True)
        if ignore not in (None, -100):             # the validation loss of the reference skips the pad id (train.py:351-354)
            y = torch.where(y == ignore, torch.full_like(y, -100), y)
        for j, d in enumerate(depths):
            pair = torch.tensor([d, 0]) if mc.is_recurrent else None
            sums[j] += model(x, labels=y, num_steps_pair=pair)["loss"].float()
        n += 1
    model.train()
    means = fabric.all_reduce(sums / max(n, 1), "mean")
    out = {f"val_loss_depth_{d}": float(v) for d, v in zip(depths, means)}
    # the reference's names: the full-depth value twice, and one pair per evaluated depth (train.py:377-383)
    out["val_loss"] = float(means[-1])
    out["val_ppl"] = math.exp(min(out["val_loss"], 30.0))
    for d, v in zip(depths, means):
        out[f"val_loss_{d}"] = float(v)
        out[f"val_ppl_{d}"] = math.exp(min(float(v), 30.0))
    return out


def _reference_metric_names(cfg, fabric, state, metrics: dict, running_loss: float, total_flops: float, t_start: float,
                            initial_step: int) -> dict:
    """The same quantities under the names the reference logs (train.py:566-636), so that dashboards built on its runs
    keep working: whole-job throughput, time bookkeeping, utilisation, memory, and the data-mixture state."""
    step = state["microbatch_step"]
    sps = max(metrics.get("steps_per_second", 0.0), 1e-12)
    elapsed = time.time() - t_start
    done = max(step - initial_step, 1)
    out = {
        "local_loss": running_loss, "local_ppl": math.exp(min(running_loss, 30.0)), "microbatch_step": step,
        "steps/second": sps, "seconds/step": 1.0 / sps,
        "tokens/second": metrics.get("tokens_per_second", 0.0) * fabric.world_size,
        "remaining_time": elapsed / done * max((cfg.max_steps or step) - step, 0), "total_time": elapsed,
        "global_grad_norm": metrics.get("grad_norm"), "global_train_ppl": math.exp(min(metrics["global_loss"], 30.0)),
    }
    if cfg.measure_utilization:
        out.update({"total_FLOPs": total_flops, "FLOP/S": metrics.get("tflops", 0.0) * fabric.world_size,
                    "model_flop_utilization": metrics.get("mfu", 0.0)})
        if fabric.device.type == "cuda":
            out["max_mem_per_gpu"] = torch.cuda.max_memory_allocated(fabric.device) / 1024 ** 3
            out["max_mem_reserved_per_gpu"] = torch.cuda.max_memory_reserved(fabric.device) / 1024 ** 3
            torch.cuda.reset_peak_memory_stats(fabric.device)
    sched = state.get("data_scheduler")
    if sched is not None and len(cfg.dataset_names) > 1:
        weights = list(sched.get_data_weights())
        samples = fabric.all_reduce(torch.tensor(sched.get_sample_count(), dtype=torch.float32, device=fabric.device),
                                    "sum").tolist()
        epochs = fabric.all_reduce(torch.tensor(sched.get_epoch_count(), dtype=torch.float32, device=fabric.device),
                                   "mean").tolist()
        total = sum(weights) or 1.0
        for i, name in enumerate(cfg.dataset_names):
            out[f"data_scheduler_weight/{name}"] = weights[i]
            out[f"data_scheduler_norm_weight/{name}"] = weights[i] / total
            out[f"data_scheduler_sample_count/{name}"] = samples[i]
            out[f"data_scheduler_epoch_count/{name}"] = epochs[i]
    return out


def check_device_waits(fabric, state) -> None:
    """Raise when a kernel of this rank timed out on a wait (a peer's flag, a pipeline barrier).  A timed-out wait in the
    gradient reduction already poisons that step's norm, so the update is skipped; the run still must not go on, because
    the ranks no longer agree on what they skipped."""
    code = fabric.device_status()
    if code:
        state["should_exit_training"] = True
        raise RuntimeError(f"a GPU kernel gave up on a bounded wait (status {code}) at micro-batch step "
                           f"{state['microbatch_step']}; resume from the last checkpoint")


def maybe_save(cfg, fabric, state, force: bool = False) -> None:
    step = state["microbatch_step"]
    # interval saves wait for the end of an accumulation window (train.py:912): the partial gradient sums are not part
    # of a checkpoint
    due = force or (cfg.save_step_interval and step % cfg.save_step_interval == 0 and step > 0
                    and not state.get("is_accumulating", False)) or (cfg.save_first_step and step == 1)
    if not due and cfg.save_n_min_before_job_done is not None and step % 32 == 0:
        left = slurm_seconds_left()
        t = fabric.all_reduce(torch.tensor([left if left is not None else 1e9], device=fabric.device), "mean")
        due = float(t) < 60 * cfg.save_n_min_before_job_done
    if due:
        state["optimizer_step"] = state["engine"].optimizer_step
        path = ckpt.save_checkpoint(fabric, state, cfg.out_dir, cfg.run_name)
        if path:
            fabric.print(f"saved checkpoint {path}")


def train(cfg, fabric, state) -> None:
    engine: TrainEngine = state["engine"]
    model, mc = state["model"], cfg.model_config
    loggers = make_loggers(cfg.logger_name, cfg.out_dir, cfg.run_name, cfg.logger_project, fabric.global_rank)
    fabric._loggers = loggers                     # fabric.log_dict / log_to_summary reach the same sinks
    warmup_or_early_fail_allreduce(fabric)
    loss_mean, timer = RunningMean(32), StepTimer()
    total_tokens, total_flops, t_start, initial_step = 0, 0.0, time.time(), state["microbatch_step"]
    tokens_per_mb = cfg.micro_batch_size * cfg.block_size
    for x, y, _meta in state["train_dataloader"]:
        if state["microbatch_step"] >= cfg.max_steps:
            break
        if cfg.goldfish.strategy is not None:
            y, _ = apply_tld(y, cfg.goldfish, ignore_index=-100)
        x, y = x.to(fabric.device, non_blocking=True), y.to(fabric.device, non_blocking=True)
        if cfg.batch_size_ramp:
            engine.grad_accum = get_batch_size(state["microbatch_step"], cfg.batch_size_ramp,
                                               cfg.batch_size // cfg.micro_batch_size)
        monitor_now = cfg.model_telemetry and (state["microbatch_step"] + 1) % max(cfg.log_step_interval, 1) == 0
        if monitor_now:
            enable_monitoring(model, True)
        if state["microbatch_step"] < cfg.shape_watching_steps:
            fabric.print(f"step {state['microbatch_step']}: input {tuple(x.shape)} labels {tuple(y.shape)}")
        out = engine.train_step(x, y)
        state["microbatch_step"] = engine.micro_step
        state["optimizer_step"] = engine.optimizer_step
        state["is_accumulating"] = engine.is_accumulating()
        n, k = out["depths"]
        flops = mc.flops_per_token(cfg.block_size, n, k) * tokens_per_mb if mc.is_recurrent else \
            mc.flops_per_token(cfg.block_size, 0, 0) * tokens_per_mb
        timer.add(tokens_per_mb, flops)
        total_tokens += tokens_per_mb * fabric.world_size
        total_flops += flops * fabric.world_size
        if state["microbatch_step"] % max(cfg.log_step_interval, 1) == 0:
            loss = float(out["loss"])  # host sync only at log points
            check_device_waits(fabric, state)
            if not math.isfinite(loss) and not cfg.allow_nonfinite_loss:
                state["should_exit_training"] = True
                fabric.print(f"non-finite loss {loss} at step {state['microbatch_step']}")
            loss_mean.update(loss)
            metrics = {"loss": loss, "loss_running": loss_mean.compute(), "lr": engine.optimizer.param_groups[0]["lr"],
                       "num_steps_no_grad": n, "num_steps_with_grad": k, "total_tokens": total_tokens,
                       "optimizer_step": engine.optimizer_step}
            if out["grad_norm"] is not None:
                metrics["grad_norm"] = float(out["grad_norm"])
            gl = fabric.all_reduce(torch.tensor([loss], device=fabric.device), "mean")
            metrics["global_loss"] = float(gl)
            if cfg.loss_guardrail_active and metrics["global_loss"] > 6 * max(loss_mean.compute(), 1e-6):
                state["should_exit_training"] = True
            metrics.update(timer.read_and_reset())
            if torch.cuda.is_available():
                metrics["peak_mem_gb"] = torch.cuda.max_memory_allocated() / 2**30
            if monitor_now:
                metrics.update(harvest_metrics(model))
                metrics.update(optimizer_telemetry(model, engine.optimizer))
                enable_monitoring(model, False)
            metrics.update(_reference_metric_names(cfg, fabric, state, metrics, loss_mean.compute(), total_flops, t_start,
                                                   initial_step))
            state["metrics"] = metrics
            for lg in loggers:
                lg.log_metrics(metrics, step=state["microbatch_step"])
            fabric.print(f"step {state['microbatch_step']:>7} | loss {loss:.4f} | lr {metrics['lr']:.2e} | "
                         f"(n,k)=({n},{k}) | {metrics['tokens_per_second']:.0f} tok/s/rank | MFU {metrics['mfu']:.3f}")
        if cfg.eval_step_interval and state["microbatch_step"] % cfg.eval_step_interval == 0:
            vm = validate(cfg, fabric, state)
            for lg in loggers:
                lg.log_metrics(vm, step=state["microbatch_step"])
            fabric.print(" | ".join(f"{k} {v:.4f}" for k, v in vm.items()))
        state["data_scheduler"].step(state["microbatch_step"])
        if state["microbatch_step"] % 32 == 0:
            # element 0: exit flag, MIN over ranks (all must ask); element 1: minus the device status word, MIN over
            # ranks = the worst status anywhere, so that every rank stops when one rank's kernels gave up on a peer
            code = fabric.device_status()
            flag = torch.tensor([1.0 if state["should_exit_training"] else 0.0, -float(code)], device=fabric.device)
            if fabric.is_distributed:
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            flag = flag.tolist()
            if flag[1] < 0:
                raise RuntimeError(f"a GPU kernel gave up on a bounded wait on some rank (status {int(-flag[1])}, "
                                   f"this rank {code}); parameters may have diverged -- resume from the last checkpoint")
            if bool(flag[0]):
                fabric.print("all ranks requested exit; stopping")
                break
        maybe_save(cfg, fabric, state)
    if cfg.save_last_step:
        maybe_save(cfg, fabric, state, force=True)


def main(cfg) -> dict:
    device_health_check()
    set_torch_flags(cfg)
    fabric = setup_fabric(cfg)
    try:
        state = startup(cfg, fabric)
        train(cfg, fabric, state)
        return state
    finally:
        fabric.shutdown()  # the process group is destroyed on every exit path
