"""Headline benchmark: training tokens/s of nebel-raven-3.5b (seq 4096, micro-batch 1 per GPU, recurrence sampled
with mean 32, truncated backprop depth 8, AdamW with global-norm clip 1.0) on N GPUs of one node.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same metric/config

Rank 0 prints ONE JSON line.  Timing: CUDA events on the launching stream around exactly K steps, bracketed by a
barrier + device synchronise on both sides, max over ranks.  The per-step working set (7.1 GB of bf16 weights
streamed per recurrence, ~30 GB of activations) is far larger than the 126 MB L2, so no explicit L2 flush is needed.
SM clocks and throttle reasons are sampled with nvidia-smi during the timed region.  A second timed region measures
the same steps end to end through the public API (``TrainEngine.train_step``) including a pinned host->device copy
of every step's tokens and a device->host read of every step's loss.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))

MODEL = "nebel-raven-3.5b"
SEQ = 4096
BASELINE_PUBLISHED = None  # the reference publishes no tokens/s figure for this config


# ------------------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while a region is being timed (read-only query)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i",
                 str(self.idx)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    mx.append(float(p[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     p[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    return rank, world, local


def max_over_ranks(value: float, device) -> float:
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return value


def sync_all(device):
    import torch
    import torch.distributed as dist

    torch.cuda.synchronize(device)
    if dist.is_available() and dist.is_initialized():
        dist.barrier(device_ids=[device.index])
    torch.cuda.synchronize(device)


def make_batches(n: int, vocab: int, seed: int, rank: int):
    """Synthetic uniform-random token rows of block_size+1, pinned in host memory (one row per step)."""
    import torch

    g = torch.Generator().manual_seed(seed + 1000 * rank)
    rows = torch.randint(0, vocab, (n, 1, SEQ + 1), generator=g, dtype=torch.int64)
    return rows.pin_memory()


def timed_region(step_fn, steps: int, device, sampler: ClockSampler | None):
    """Device time in ms for `steps` calls of step_fn(i), max over ranks."""
    import torch

    sync_all(device)
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(i)
    e1.record()
    sync_all(device)
    clocks = sampler.stop() if sampler else None
    return max_over_ranks(e0.elapsed_time(e1), device), clocks


# ------------------------------------------------------------------------------------------------------
def device_mem_used_gb(device) -> float:
    """Device memory in use as the driver sees it (symmetric buffers come from cudaMalloc, outside torch's allocator)."""
    import torch

    free, total = torch.cuda.mem_get_info(device)
    return round((total - free) / 2**30, 1)


def build_engine(args, sync: str, fixed_depth: bool, grad_accum: int):
    import torch

    from recurrent_pretraining_b200.config import ModelConfig
    from recurrent_pretraining_b200.parallel.fabric import Fabric
    from recurrent_pretraining_b200.runtime.engine import TrainEngine

    fabric = Fabric.from_env(grad_sync=sync)
    over = dict(lockstep_n=True, lockstep_k=True)
    if fixed_depth:
        over["sampling_scheme"] = "fixed"
    cfg = ModelConfig.from_name(args.model, **over)
    torch.manual_seed(1337)
    with torch.device(fabric.device):
        model = cfg.construct_model()
    flags = dict(atan2=True, update_clipping=True, running_init=True, decouple_wd=True) \
        if args.optimizer == "ellis" else {}
    engine = TrainEngine(model, fabric, lr=4e-4, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8, grad_clip=1.0,
                         grad_accum=grad_accum, **flags)
    return fabric, cfg, engine


def decode_block(args, device) -> dict:
    """Decode throughput of the native engine on this GPU (one replica): prompt 512 uniform-random tokens, 256 new
    tokens, greedy, fixed r = 32 at batch 1/8/32/64, and the KL-exit variant (5e-4, at most 64 recurrences, latent
    reuse) at batch 1/8/32.  Device-timed; prefill excluded and reported."""
    import torch

    from recurrent_pretraining_b200.engine.decode import DecodeEngine
    from recurrent_pretraining_b200.utils.decode_bench import build_model, time_region

    prompt, new = 512, int(os.environ.get("B200_BENCH_DECODE_NEW", "256"))
    model = build_model(args.model)
    V = model.config.padded_vocab_size
    hbm = None
    try:
        hbm = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
    except Exception:
        pass
    out = {"prompt": prompt, "new_tokens": new, "greedy": True, "hbm_copy_peak_gbs": hbm, "fixed_r32": {}, "kl_exit": {}}
    for tag, batches, kw, max_steps in (("fixed_r32", (1, 8, 32, 64), {}, 32),
                                        ("kl_exit", (1, 8, 32),
                                         dict(criterion="kl", exit_threshold=5e-4, max_steps=64, continuous_compute=True), 64)):
        for B in batches:
            try:
                ids = torch.randint(0, V - 100, (B, prompt), device=device)
                eng = DecodeEngine(model, B, prompt + new + 1, num_steps=32, max_steps=max_steps)
                eng.generate(ids, 4, **kw)                       # warm-up: graph capture
                t_pre, _ = time_region(lambda: eng.prefill(ids, 32))
                t_all, (_, stats) = time_region(lambda: eng.generate(ids, new, **kw))
                t_dec = t_all - t_pre
                mean_r = sum(sum(x) for x in stats["steps"]) / max(1, B * len(stats["steps"]))
                gbs = eng.weight_bytes_per_recurrence * mean_r / (t_dec / (new - 1)) / 1e6
                out[tag][str(B)] = {"tok_s": round(B * (new - 1) / (t_dec / 1e3), 1),
                                    "ms_per_token": round(t_dec / (new - 1), 2), "prefill_ms": round(t_pre, 1),
                                    "mean_recurrence": round(mean_r, 2), "weight_stream_gbs": round(gbs),
                                    "frac_of_hbm_copy_peak": round(gbs / hbm, 3) if hbm else None,
                                    "kv_cache_gib": round(eng.cache.get_memory_usage() / 1024, 1),
                                    "device_status": stats["device_status"]}
                del eng
            except Exception as exc:  # noqa: BLE001  (an out-of-memory batch must not lose the other rows)
                out[tag][str(B)] = {"error": f"{type(exc).__name__}: {exc}"[:160]}
            torch.cuda.empty_cache()
    return out


def run_steps(engine, args, device, rank, local, world, micro_per_step: int):
    """Warm-up, the device-timed region and the end-to-end region of one engine; returns the record pieces."""
    import torch

    from recurrent_pretraining_b200.ops import cuda as C

    total = (args.warmup + args.steps) * micro_per_step
    vocab = engine.model.config.padded_vocab_size
    host = make_batches(total, vocab, 0, rank)
    dev_rows = host.to(device)

    def device_step(i, base):
        for j in range(micro_per_step):
            row = dev_rows[(base + i) * micro_per_step + j]
            engine.train_step(row[:, :-1], row[:, 1:])

    for i in range(args.warmup):
        device_step(i, 0)
    start_micro, start_opt = engine.micro_step, engine.optimizer_step
    launches0 = C.launch_count()
    ms, clocks = timed_region(lambda i: device_step(i, args.warmup), args.steps, device, ClockSampler(local))
    launches = C.launch_count() - launches0
    status = C.check_device_status()
    # end-to-end region: same step indices (same sampled recurrence depths), inputs from pinned host memory
    engine.micro_step, engine.optimizer_step = start_micro, start_opt
    losses, norms = [], []

    def e2e_step(i):
        for j in range(micro_per_step):
            row = host[(args.warmup + i) * micro_per_step + j].to(device, non_blocking=True)
            out = engine.train_step(row[:, :-1], row[:, 1:])
            losses.append(float(out["loss"].item()))
            if out["grad_norm"] is not None:
                norms.append(out["grad_norm"])

    ms_e2e, _ = timed_region(e2e_step, args.steps, device, None)
    tokens = world * SEQ * args.steps * micro_per_step
    return {"ms": ms, "ms_e2e": ms_e2e, "tokens": tokens, "clocks": clocks, "launches": launches, "status": status,
            "final_loss": losses[-1] if losses else None,
            "final_grad_norm": float(norms[-1]) if norms else None, "host": host}


def run_ours(args):
    import torch

    os.environ.setdefault("B200_TRACE", "1")    # CUDA-event stamps of the bucket reductions (a few events per step)
    rank, world, local = dist_env()
    zero3 = args.mode == "zero3"
    accum = 8 if zero3 else 1
    sync = "zero3" if zero3 else os.environ.get("B200_GRAD_SYNC", "p2p")
    fabric, cfg, engine = build_engine(args, sync, fixed_depth=zero3, grad_accum=accum)
    device = fabric.device
    r = run_steps(engine, args, device, rank, local, world, accum)
    value = r["tokens"] / (r["ms"] / 1e3)
    stepper = getattr(fabric, "_p2p", None)
    metric = "train tokens/sec (raven-3.5B, r=32 mean sampled, bptt 8)" if not zero3 else \
        "train tokens/sec (raven-3.5B, r=32 fixed, bptt 8, params/grads/optimizer sharded, accumulation 8)"
    rec = {
        "metric": metric, "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(r["ms"] / args.steps, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": (value / BASELINE_PUBLISHED) if BASELINE_PUBLISHED else None,
        "dtype": "bf16 compute (weights, activations, GEMMs); fp32 master weights, gradients and optimizer state",
        "data": "synthetic uniform-random tokens, random-init weights", "impl": "ours",
        "config": {"model": args.model, "global_batch": world * accum, "seq_len": SEQ,
                   "parallelism": f"dp{world}" + ("-zero3" if zero3 else ""),
                   "micro_batch": 1, "grad_accum": accum, "mean_recurrence": cfg.mean_recurrence,
                   "backprop_depth": cfg.mean_backprop_depth, "sampling": cfg.sampling_scheme,
                   "optimizer": "AdamW fused, clip 1.0" if args.optimizer == "adamw" else
                   "ELLISAdam flags (update clipping, atan2, running init, decoupled decay) fused, clip 1.0",
                   "grad_sync": fabric.grad_sync if world > 1 else "none",
                   "overlap": bool(stepper is not None and stepper.overlap),
                   "param_sync": ("pull in the next forward pass" if stepper.zero3 else "push from the update kernel")
                   if stepper is not None else "none",
                   "l2": "working set (7.1 GB weights per recurrence) >> 126 MB L2; no explicit flush",
                   "activation_checkpointing": False},
        "clocks": r["clocks"],
        "e2e": {"value": round(r["tokens"] / (r["ms_e2e"] / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": (SEQ + 1) * 8 * accum, "d2h_bytes_per_step": 4 * accum},
        "gpu_launches": r["launches"], "device_status": r["status"],
        "final_loss": r["final_loss"], "final_grad_norm": r["final_grad_norm"],
        "peak_mem_gb": round(torch.cuda.max_memory_allocated(device) / 2**30, 1),
        "device_mem_used_gb": device_mem_used_gb(device),
    }
    from recurrent_pretraining_b200.ops import cuda as _K

    rec["library_calls"] = dict(_K.LIBRARY_CALLS)     # declared library paths taken by the timed steps (none expected)
    # ---- evidence blocks outside the timed regions; a failure here never loses the headline line
    if stepper is not None and os.environ.get("B200_BENCH_EXTRAS", "1") == "1":
        try:
            rec["persistent_bytes_per_rank"] = stepper.persistent_bytes()
            if stepper.tracing:
                rec["timeline_ms"] = stepper.timeline()
            rec["replicas_identical"] = stepper.replicas_identical()
            engine._begin_window()
            engine.model._phase_cb = None
            engine.model.step = engine.micro_step + 1
            row = r["host"][0].to(device)
            engine.model(row[:, :-1], labels=row[:, 1:])["loss"].backward()
            rec["grad_rel_err_vs_nccl"] = max_over_ranks(stepper.reduce_check(), device)
            if stepper.last_check:
                rec["grad_check_worst"] = sorted(stepper.last_check, key=lambda x: -x[1])[:4]
        except Exception as exc:  # noqa: BLE001
            rec["consistency_error"] = f"{type(exc).__name__}: {exc}"[:200]
    fabric_closed = False
    if world == 1 and not zero3 and os.environ.get("B200_BENCH_DECODE", "1") == "1" and args.model == MODEL:
        try:
            import gc

            from recurrent_pretraining_b200.ops import cuda as C

            engine.optimizer = engine.model = None       # the flat buffers, the optimizer state and the scratch
            fabric.flat_groups = []                      # tensors go back before the KV caches are sized
            C._ce_scratch.clear()
            del engine, r
            gc.collect()
            torch.cuda.empty_cache()
            rec["device_mem_used_before_decode_gb"] = device_mem_used_gb(device)
            rec["decode"] = decode_block(args, device)
        except Exception as exc:  # noqa: BLE001
            rec["decode"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if not fabric_closed:
        fabric.shutdown()


# ------------------------------------------------------------------------------------------------------
def run_reference(args):
    """The unmodified reference (baseline/_ref): its RecurrentGPT, SimpleFabric (bf16-mixed autocast wrapper,
    chunked NCCL all-reduce inside ``fabric.backward``), its optimizer factory (torch AdamW, fused) and its
    clip_gradients -- the train_step sequence of the reference's train.py:389-475."""
    try:
        import refload

        if not refload.available():
            raise ImportError("baseline/_ref is empty (reference not installed)")
        import torch

        rank, world, local = dist_env()
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        os.environ.setdefault("LOCAL_RANK", "0")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        utils = refload.module("utils")
        optim = refload.module("optim")
        fabric = utils.SimpleFabric(precision="bf16-mixed")
        device = fabric.device
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {exc}"[:300]}), flush=True)
        return

    def build(checkpointing: bool, compiled: bool = False):
        torch.manual_seed(1337)
        with torch.device(device):
            model, cfg = refload.build_train_model(args.model, gradient_checkpointing=checkpointing,
                                                   lockstep_n=True, lockstep_k=True, attn_impl="sdpa")
        model = fabric.setup(model, compile=compiled)
        groups = optim.get_param_groups(model.named_parameters(), no_weight_decay_for_bias_and_norm_params=False)
        opt = optim.get_optimizer("AdamW")(groups, lr=4e-4, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8)
        return model, cfg, opt

    # The reference's own launch configs train with ``compile_model: true`` (its fabric.setup wraps the model in
    # torch.compile, max-autotune without CUDA graphs); that is the arm's default.  REF_COMPILE=0 gives the eager arm; a
    # compile failure during warm-up falls back to eager and is recorded.
    state = {"checkpointing": os.environ.get("REF_CHECKPOINT", "0") == "1",
             "compile": os.environ.get("REF_COMPILE", "1") == "1", "compile_fallback": None}
    model, cfg, opt = build(state["checkpointing"], state["compile"])
    total = args.warmup + args.steps
    host = make_batches(total, cfg.padded_vocab_size, 0, rank)
    dev_rows = host.to(device)
    counters = {"micro": 0, "opt": 0}
    last_norm = [None]

    def train_step(input_ids, labels):
        counters["micro"] += 1
        inner = model.module if hasattr(model, "module") else model
        inner.step = counters["micro"]
        out = model(input_ids, position_ids=None, labels=labels, attention_mask=None)
        loss = out["loss"]
        fabric.backward(loss, model=model)
        for g in opt.param_groups:
            g["lr"] = torch.tensor(4e-4 * g["base_lr"], device=device)
        gn = fabric.clip_gradients(model, opt, max_norm=1.0)
        last_norm[0] = gn
        if torch.isfinite(gn) and counters["opt"] > 0:
            opt.step()
        opt.zero_grad(set_to_none=False)
        counters["opt"] += 1
        return loss

    def device_step(i, base):
        row = dev_rows[base + i]
        train_step(row[:, :-1], row[:, 1:])

    try:
        for i in range(args.warmup):
            device_step(i, 0)
    except torch.cuda.OutOfMemoryError:
        del model, opt
        torch.cuda.empty_cache()
        state["checkpointing"] = True
        model, cfg, opt = build(True, state["compile"])
        counters.update(micro=0, opt=0)
        for i in range(args.warmup):
            device_step(i, 0)
    except Exception as exc:  # noqa: BLE001
        if not state["compile"]:
            raise
        state["compile"], state["compile_fallback"] = False, f"{type(exc).__name__}: {exc}"[:200]
        del model, opt
        torch.cuda.empty_cache()
        model, cfg, opt = build(state["checkpointing"], False)
        counters.update(micro=0, opt=0)
        for i in range(args.warmup):
            device_step(i, 0)
    start = dict(counters)
    ms, clocks = timed_region(lambda i: device_step(i, args.warmup), args.steps, device, ClockSampler(local))
    counters.update(start)
    losses, norms = [], []

    def e2e_step(i):
        row = host[args.warmup + i].to(device, non_blocking=True)
        losses.append(float(train_step(row[:, :-1], row[:, 1:]).item()))
        norms.append(last_norm[0])

    ms_e2e, _ = timed_region(e2e_step, args.steps, device, None)
    tokens = world * SEQ * args.steps
    rec = {
        "metric": "train tokens/sec (raven-3.5B, r=32 mean sampled, bptt 8)", "value": round(tokens / (ms / 1e3), 1),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 autocast, fp32 master weights", "data": "synthetic uniform-random tokens, random-init weights",
        "impl": "reference",
        "config": {"model": args.model, "global_batch": world, "seq_len": SEQ, "parallelism": f"dp{world}",
                   "micro_batch": 1, "attn_impl": "sdpa", "compile": state["compile"],
                   "compile_fallback": state["compile_fallback"],
                   "activation_checkpointing": state["checkpointing"],
                   "l2": "working set >> 126 MB L2; no explicit flush"},
        "clocks": clocks,
        "e2e": {"value": round(tokens / (ms_e2e / 1e3), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": (SEQ + 1) * 8, "d2h_bytes_per_step": 4},
        "final_loss": losses[-1] if losses else None,
        "final_grad_norm": float(norms[-1]) if norms and norms[-1] is not None else None,
        "peak_mem_gb": round(torch.cuda.max_memory_allocated(device) / 2**30, 1),
    }
    if world == 1 and os.environ.get("B200_BENCH_DECODE", "1") == "1" and args.model == MODEL:
        try:
            del model, opt
            import gc

            gc.collect()
            torch.cuda.empty_cache()
            rec["decode"] = reference_decode_block(refload, device)
        except Exception as exc:  # noqa: BLE001
            rec["decode"] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    if rank == 0:
        print(json.dumps(rec), flush=True)
    try:
        torch.distributed.destroy_process_group()
    except Exception:
        pass


def reference_decode_block(refload, device) -> dict:
    """Decode throughput of the unmodified reference HF model (raven_modeling_minimal.py): prompt 512, greedy, r = 32,
    its own HuginnDynamicCache, driven token by token through ``forward`` (its ``generate`` does not run under the
    installed transformers); batch 1 and 8, 16 timed tokens after a 2-token warm-up."""
    import torch

    mod = refload.module("raven_modeling_minimal")
    mod.RavenForCausalLM._tied_weights_keys = {"lm_head.weight": "transformer.wte.weight"}
    cfgmod = refload.module("raven_config_minimal")
    torch.manual_seed(0)
    with torch.device(device):
        model = mod.RavenForCausalLM(cfgmod.RavenConfig()).to(torch.bfloat16).eval()
    V, prompt, warm, n = model.config.padded_vocab_size, 512, 2, 16
    out = {"prompt": prompt, "timed_tokens": n, "greedy": True, "r": 32, "fixed_r32": {}}
    for B in (1, 8):
        ids = torch.randint(0, V - 100, (B, prompt), device=device)
        with torch.no_grad():
            cache = mod.HuginnDynamicCache()
            o = model(ids, num_steps=32, use_cache=True, past_key_values=cache,
                      cache_position=torch.arange(prompt, device=device))
            tok = o.logits[:, -1].argmax(-1, keepdim=True)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for t in range(warm + n):
                if t == warm:
                    torch.cuda.synchronize(device)
                    e0.record()
                o = model(tok, num_steps=32, use_cache=True, past_key_values=cache,
                          cache_position=torch.tensor([prompt + t], device=device))
                tok = o.logits[:, -1].argmax(-1, keepdim=True)
            e1.record()
            torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1)
        out["fixed_r32"][str(B)] = {"tok_s": round(B * n / (ms / 1e3), 2), "ms_per_token": round(ms / n, 1)}
        del cache
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--mode", default="dp", choices=["dp", "zero3"],
                    help="dp: the headline data-parallel config; zero3: fixed r=32, k=8, accumulation 8, parameters, "
                         "gradients and optimizer state sharded over the GPUs (needs >= 2 GPUs)")
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "ellis"],
                    help="adamw: the headline config; ellis: the reference's production optimizer flags on the same path")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.model == MODEL else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
