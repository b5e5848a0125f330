"""Checkpoint save / resume in the reference's layout.

Path: ``{out_dir}/{prefix}/step-{microbatch_step:08d}-{run_name}_{local_rank}.pth`` with ``prefix =
checkpoints-sane-ddp`` (train.py:905-933, recpre/utils.py:1208-1241).  Only the ranks of node 0 write, one file per
local rank (optimizer state is sharded per rank); every rank still builds its state so that collectives inside
``state_dict`` (dataset state gather, master-weight gather) stay matched.  The file is a ``torch.save`` of a dict:
``model`` (inner state-dict keys ``transformer.*``, ``lm_head.weight``, ``freqs_cis``; optionally also under the
``_original_module.`` / ``_forward_module.`` prefixes the reference's wrapper produces), ``optimizer``,
``train_dataloader``, ``data_scheduler``, the step counters, ``metrics``, ``should_exit_training`` and the
``model_config`` dict.  Loading picks the newest step for the run name and strips any wrapper prefixes.
"""
from __future__ import annotations

import glob
import os
import re

import torch

PREFIX = "checkpoints-sane-ddp"
_WRAPPER_PREFIXES = ("_orig_mod.", "_original_module.", "_forward_module.", "module.")


def strip_wrapper_prefixes(sd: dict) -> dict:
    """Map a (possibly wrapped / compiled / duplicated) model state dict to inner-module keys."""
    out = {}
    for k, v in sd.items():
        changed = True
        while changed:
            changed = False
            for p in _WRAPPER_PREFIXES:
                if k.startswith(p):
                    k, changed = k[len(p):], True
        out.setdefault(k, v)
    return out


def checkpoint_dir(out_dir: str) -> str:
    return os.path.join(out_dir, PREFIX)


def checkpoint_stem(out_dir: str, run_name: str, microbatch_step: int) -> str:
    return os.path.join(checkpoint_dir(out_dir), f"step-{microbatch_step:08d}-{run_name}")


def model_state_dict(model, reference_prefixes: bool = False, engine=None) -> dict:
    if engine is not None and hasattr(engine, "model_state_dict") and getattr(engine, "mode", "") == "fused":
        sd = engine.model_state_dict()     # reassembles fp32 masters that exist only as per-rank pieces
    else:
        sd = {k: v.detach().to("cpu", copy=True) if torch.is_tensor(v) else v for k, v in model.state_dict().items()}
    sd = {k: (v.float() if torch.is_tensor(v) and v.dtype == torch.bfloat16 and k != "freqs_cis" else v)
          for k, v in sd.items()}
    if reference_prefixes:
        dup = {}
        for k, v in sd.items():
            dup["_forward_module." + k] = v
            dup["_original_module." + k] = v
        return dup
    return sd


def save_checkpoint(fabric, state: dict, out_dir: str, run_name: str, reference_prefixes: bool = False,
                    local_devices: int | None = None) -> str | None:
    """``state`` holds live objects: model, engine (optimizer + counters), train_dataloader, data_scheduler, plus plain
    values.  Returns the written path (None on ranks that do not write)."""
    engine = state.get("engine")
    payload = {}
    for key, value in state.items():
        if key == "model":
            # collective on the sharded paths: stale or sharded fp32 masters are completed from their owners
            payload[key] = model_state_dict(value, reference_prefixes, engine)
        elif key == "engine":
            payload["optimizer"] = [value.state_dict()]
        elif key in ("train_dataloader", "data_scheduler") and value is not None:
            payload[key] = value.state_dict()
        elif key in ("tokenizer", "val_dataloader"):
            continue
        else:
            payload[key] = value
    local_devices = local_devices or int(os.getenv("LOCAL_WORLD_SIZE", os.getenv("SLURM_NTASKS_PER_NODE",
                                                                                 max(torch.cuda.device_count(), 1))))
    if fabric.global_rank >= min(local_devices, fabric.world_size):
        return None
    os.makedirs(checkpoint_dir(out_dir), exist_ok=True)
    path = f"{checkpoint_stem(out_dir, run_name, state['microbatch_step'])}_{fabric.local_rank}.pth"
    tmp = path + ".tmp"
    torch.save(payload, tmp)
    os.replace(tmp, path)  # a crash mid-write never leaves a truncated file under the final name
    return path


def find_latest(out_dir: str, run_name: str, local_rank: int) -> str | None:
    """Newest checkpoint file of the run for this local rank; when the run was saved by fewer ranks (resume on a
    larger world), the newest file of rank 0."""
    for rank in (local_rank, 0):
        best, best_step = None, -1
        for p in glob.glob(os.path.join(checkpoint_dir(out_dir), f"step-*-{run_name}_{rank}.pth")):
            m = re.search(r"step-(\d+)-", os.path.basename(p))
            if m and int(m.group(1)) > best_step:
                best, best_step = p, int(m.group(1))
        if best is not None:
            return best
    return None


def sibling_paths(path: str) -> list:
    """All per-rank files of the checkpoint that ``path`` belongs to, ordered by the rank suffix."""
    m = re.match(r"(.*)_(\d+)\.pth$", path)
    if not m:
        return [path]
    found = []
    for p in glob.glob(m.group(1) + "_*.pth"):
        mm = re.match(r".*_(\d+)\.pth$", p)
        if mm:
            found.append((int(mm.group(1)), p))
    return [p for _, p in sorted(found)]


def load_checkpoint(fabric, state: dict, path: str, strict: bool = True) -> dict:
    """``path`` is this rank's file; when the world size changed since the save and no file exists for this rank,
    pass any rank's file: model, counters and loader state are identical in all of them, and the sharded optimizer
    state is re-cut from the whole set of files."""
    ckpt = torch.load(path, map_location="cpu", weights_only=False)

    def all_engine_states():
        out = []
        for p in sibling_paths(path):
            other = ckpt if p == path else torch.load(p, map_location="cpu", weights_only=False)
            opt = other["optimizer"]
            out.append(opt[0] if isinstance(opt, list) else opt)
        return out

    for key, value in ckpt.items():
        if key == "model":
            sd = strip_wrapper_prefixes(value)
            engine = state.get("engine")
            if engine is not None and getattr(engine, "mode", "") == "fused":
                engine.load_model_state(sd, strict)
                continue
            model = state["model"]
            own = model.state_dict()
            with torch.no_grad():
                for k, v in sd.items():
                    if k in own:
                        own[k].copy_(v.to(own[k].dtype))
                    elif strict and k != "lm_head.weight":
                        raise KeyError(f"unexpected key {k} in checkpoint")
            missing = [k for k in own if k not in sd and not (k == "lm_head.weight")]
            if strict and missing:
                raise KeyError(f"missing keys in checkpoint: {missing[:5]}")
        elif key == "optimizer":
            if state.get("engine") is not None:
                state["engine"].load_state_dict(value[0] if isinstance(value, list) else value,
                                                other_shards=all_engine_states)
        elif key in ("train_dataloader", "data_scheduler"):
            if state.get(key) is not None:
                state[key].load_state_dict(value)
        elif key in ("tokenizer", "val_dataloader"):
            continue
        else:
            state[key] = value
    if state.get("engine") is not None:
        state["engine"].refresh_shadows()
    return ckpt
