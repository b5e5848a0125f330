#!/usr/bin/env python
"""Self-contained supervised finetuning of the HF-style recurrent model (`RavenForCausalLM`).

Data-parallel over the ranks of `torch.distributed.run` (one process per GPU; CPU/gloo works for smoke runs), gradient
accumulation without inter-rank traffic on the non-final micro-steps, warmup-stable-decay schedule, loss on assistant
tokens only for chat-formatted data.  Functional counterpart of the reference's finetuning_simple_example.py
(:61-93 settings, :186-227 chat formatting with assistant mask, :287-302 schedule, :319-390 training loop).

There is no network here, so the dataset is a local file: a `.jsonl` / `.parquet` with question / answer columns, or
`--dataset_location synthetic` for generated arithmetic questions (the smoke path of the tests).

    python finetuning_simple_example.py --model_name tiny --dataset_location synthetic --max_steps 4
    python -m torch.distributed.run --nproc-per-node 8 finetuning_simple_example.py --model_name /path/to/hf_folder \
        --dataset_location data/gsm8k_train.jsonl --batch_size 32 --micro_batch_size 2
"""
from __future__ import annotations

import argparse
import json
import math
import os
import random
import time
from dataclasses import asdict, dataclass, field
from typing import Any, Optional

import torch

from recurrent_pretraining_b200.models.hf import RavenForCausalLM
from recurrent_pretraining_b200.models.hf_config import RavenConfig
from recurrent_pretraining_b200.parallel.fabric import Fabric

DEFAULT_SYS_PROMPT = "You are a helpful assistant that can assist users with mathematical reasoning."
ASSISTANT_ROLE = "Huginn"


@dataclass
class CLISettings:
    run_name: str = "default-run"
    out_path: str = "outputs"
    dataset_location: str = "synthetic"
    model_name: str = "tiny"                 # "tiny" | a registry shape name | a local HF folder
    tokenizer_path: Optional[str] = None     # local tokenizer folder; None = byte-level fallback
    dataset_args: dict[str, Any] = field(default_factory=lambda: dict(q_col="question", a_col="answer"))
    dataset_config: str = "main"             # configuration / sub-folder of a dataset saved with the `datasets` package
    max_seq_length: int = 128
    max_samples: Optional[int] = None
    micro_batch_size: int = 2
    compile: bool = False                    # accepted for command-line compatibility: the kernels are built ahead of time
    max_steps: int = 0
    epochs: int = 1
    batch_size: int = 32
    optim_config: dict[str, Any] = field(default_factory=lambda: dict(lr=5e-7, weight_decay=0.0, betas=(0.9, 0.95),
                                                                       eps=1e-8))
    scheduler_args: dict[str, Any] = field(default_factory=lambda: dict(warmup=0.1, cooldown=0.1, min_lr_ratio=0.001))
    eval_interval: int = 1_000_000_000       # optimizer steps between validations on the held-out rows
    seed: int = 74
    take_loss_over_all_tokens: bool = False
    max_grad_norm: float = 1_000_000.0
    precision: str = "bf16-true"
    gradient_checkpointing: bool = False
    num_steps: Optional[int] = None          # fixed recurrence for training; None = sampled (n, k) as in pretraining
    save_final_checkpoint: bool = False


# ---------------------------------------------------------------------------------------------- tokenisation
class ByteTokenizer:
    """Fallback when no tokenizer folder is given: bytes + a few role markers (ids ≥ 256)."""

    bos, eos, pad, sys_id, user_id, asst_id, end_turn = 256, 257, 258, 259, 260, 261, 262
    vocab_size = 263

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def chat(self, question: str, answer: str) -> tuple[list[int], list[int]]:
        """ids and assistant mask (1 where the loss applies)."""
        pre = [self.bos, self.sys_id] + self.encode(DEFAULT_SYS_PROMPT) + [self.end_turn, self.user_id] + \
            self.encode(question) + [self.end_turn, self.asst_id]
        ans = self.encode(answer) + [self.end_turn, self.eos]
        return pre + ans, [0] * len(pre) + [1] * len(ans)


class HFChatTokenizer:
    def __init__(self, path: str):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path)
        self.pad = self.tok.pad_token_id if self.tok.pad_token_id is not None else 0
        self.vocab_size = len(self.tok)

    def chat(self, question: str, answer: str):
        msgs = [dict(role="system", content=DEFAULT_SYS_PROMPT), dict(role="user", content=question.strip()),
                dict(role=ASSISTANT_ROLE, content=answer.strip())]
        enc = self.tok.apply_chat_template(msgs, tokenize=True, add_generation_prompt=False,
                                           return_assistant_tokens_mask=True, return_dict=True)
        return list(enc["input_ids"]), list(enc.get("assistant_masks", [1] * len(enc["input_ids"])))


def load_rows(cfg: CLISettings) -> list[tuple[str, str]]:
    q, a = cfg.dataset_args["q_col"], cfg.dataset_args["a_col"]
    loc = cfg.dataset_location
    if loc == "synthetic":
        rng = random.Random(cfg.seed)
        rows = []
        for _ in range(cfg.max_samples or 256):
            x, y = rng.randint(0, 99), rng.randint(0, 99)
            rows.append((f"What is {x} plus {y}?", f"{x} + {y} = {x + y}. The answer is {x + y}."))
        return rows
    if loc.endswith(".jsonl"):
        with open(loc) as f:
            rows = [(r[q], r[a]) for r in map(json.loads, f)]
    elif loc.endswith(".parquet"):
        import pyarrow.parquet as pq

        t = pq.read_table(loc, columns=[q, a]).to_pydict()
        rows = list(zip(t[q], t[a]))
    elif os.path.isdir(loc):                 # a dataset written by `datasets.save_to_disk` (optionally per config)
        from datasets import load_from_disk

        sub = os.path.join(loc, cfg.dataset_config)
        ds = load_from_disk(sub if os.path.isdir(sub) else loc)
        ds = ds["train"] if hasattr(ds, "keys") and "train" in ds.keys() else ds
        rows = list(zip(ds[q], ds[a]))
    else:
        raise ValueError(f"dataset_location must be 'synthetic', a .jsonl / .parquet file or a saved dataset folder, "
                         f"got {loc!r}")
    return rows[: cfg.max_samples] if cfg.max_samples else rows


def tokenize(rows, tok, cfg: CLISettings):
    L = cfg.max_seq_length + 1
    ids = torch.full((len(rows), L), tok.pad, dtype=torch.long)
    mask = torch.zeros((len(rows), L), dtype=torch.bool)
    for i, (question, answer) in enumerate(rows):
        t, m = tok.chat(question, answer)
        t, m = t[:L], m[:L]
        ids[i, :len(t)] = torch.tensor(t)
        mask[i, :len(t)] = torch.tensor(m, dtype=torch.bool) if not cfg.take_loss_over_all_tokens else True
    return ids, mask


# ---------------------------------------------------------------------------------------------- model / schedule
def build_model(cfg: CLISettings, vocab_size: int, device, dtype):
    if os.path.isdir(cfg.model_name):
        model = RavenForCausalLM.from_pretrained(cfg.model_name, torch_dtype=dtype)
    else:
        if cfg.model_name == "tiny":
            hc = RavenConfig(n_embd=128, n_heads=4, n_layers=4, block_size=cfg.max_seq_length, vocab_size=max(vocab_size, 512),
                             intermediate_size=256, n_layers_in_recurrent_block=2, n_layers_in_prelude=1,
                             n_layers_in_coda=1, mean_recurrence=4, mean_backprop_depth=2)
        else:
            from recurrent_pretraining_b200.config import ModelConfig

            hc = RavenConfig.from_model_config(ModelConfig.from_name(cfg.model_name))
        torch.manual_seed(cfg.seed)
        model = RavenForCausalLM(hc).to(dtype)
    return model.to(device)


def wsd_lr(step: int, total: int, base_lr: float, warmup: float, cooldown: float, min_lr_ratio: float) -> float:
    """Warmup-stable-decay: linear up over `warmup`·total, flat, linear down to min_lr_ratio·lr over `cooldown`·total."""
    w, c = math.ceil(warmup * total), math.ceil(cooldown * total)
    if step < w:
        return base_lr * (step + 1) / max(w, 1)
    if step >= total - c:
        frac = (total - step) / max(c, 1)
        return base_lr * (min_lr_ratio + (1 - min_lr_ratio) * max(frac, 0.0))
    return base_lr


# ---------------------------------------------------------------------------------------------- training
@torch.no_grad()
def validate(model, ids, mask, cfg: CLISettings, device) -> dict:
    """Held-out loss and perplexity over the supervised positions (the reference runs an lm-eval task here,
    finetuning_simple_example.py:398-428; that package is optional, the loss is always available)."""
    was_training = model.training
    model.eval()
    total, count = 0.0, 0
    for b in range(0, len(ids), cfg.micro_batch_size):
        x = ids[b:b + cfg.micro_batch_size].to(device)
        m = mask[b:b + cfg.micro_batch_size]
        labels = torch.where(m, ids[b:b + cfg.micro_batch_size], torch.full_like(m, -100, dtype=torch.long))[:, 1:]
        n = int((labels != -100).sum())
        if n == 0:
            continue
        out = model(x[:, :-1], labels=labels.contiguous().to(device), num_steps=cfg.num_steps)
        total += float(out.loss) * n
        count += n
    model.train(was_training)
    loss = total / max(count, 1)
    return {"val_loss": loss, "val_ppl": math.exp(min(loss, 30.0)), "val_tokens": count}


def train(cfg: CLISettings) -> dict:
    fabric = Fabric.from_env(grad_sync="flat") if "RANK" in os.environ else Fabric.single(
        torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu"))
    device = fabric.device
    dtype = torch.bfloat16 if cfg.precision == "bf16-true" and device.type == "cuda" else torch.float32
    tok = HFChatTokenizer(cfg.tokenizer_path) if cfg.tokenizer_path else ByteTokenizer()
    ids, mask = tokenize(load_rows(cfg), tok, cfg)
    held = max(1, len(ids) // 20) if cfg.eval_interval < 1_000_000_000 else 0       # last 5 % of the rows
    val_ids, val_mask = ids[len(ids) - held:], mask[len(mask) - held:]
    ids, mask = ids[: len(ids) - held], mask[: len(mask) - held]
    ids, mask = ids[fabric.global_rank::fabric.world_size], mask[fabric.global_rank::fabric.world_size]
    model = build_model(cfg, tok.vocab_size, device, dtype)
    model.train()
    if cfg.gradient_checkpointing:
        model.gradient_checkpointing = True
        if hasattr(model, "gradient_checkpointing_enable"):
            try:
                model.gradient_checkpointing_enable()
            except Exception:
                pass
    validations = []
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, **{k: (tuple(v) if isinstance(v, list) else v) for k, v in cfg.optim_config.items()})
    accumulation = max(1, cfg.batch_size // (cfg.micro_batch_size * fabric.world_size))
    micro_per_epoch = len(ids) // cfg.micro_batch_size
    total_steps = cfg.max_steps or max(1, cfg.epochs * math.ceil(micro_per_epoch / accumulation))
    gen = torch.Generator().manual_seed(cfg.seed)
    step, micro, losses, t0 = 0, 0, [], time.time()
    while step < total_steps:
        order = torch.randperm(len(ids), generator=gen)
        for b in range(0, len(order) - cfg.micro_batch_size + 1, cfg.micro_batch_size):
            rows = order[b:b + cfg.micro_batch_size]
            x = ids[rows].to(device)
            labels = torch.where(mask[rows], ids[rows], torch.full_like(ids[rows], -100))[:, 1:].to(device)
            out = model(x[:, :-1], labels=labels.contiguous(), num_steps=cfg.num_steps)
            (out.loss / accumulation).backward()
            micro += 1
            if micro % accumulation:
                continue  # accumulate locally; ranks talk only on the last micro-step
            fabric.all_reduce_gradients(params)
            norm = torch.nn.utils.clip_grad_norm_(params, cfg.max_grad_norm)
            lr = wsd_lr(step, total_steps, cfg.optim_config["lr"], **cfg.scheduler_args)
            for g in opt.param_groups:
                g["lr"] = lr
            opt.step()
            opt.zero_grad(set_to_none=True)
            loss = fabric.all_reduce(out.loss.detach().float(), "mean").item()
            losses.append(loss)
            fabric.print(f"step {step:5d} | loss {loss:7.4f} | grad norm {float(norm):8.3f} | lr {lr:.3e} | "
                         f"{time.time() - t0:6.1f}s")
            step += 1
            if held and step % cfg.eval_interval == 0:
                vm = validate(model, val_ids, val_mask, cfg, device)
                validations.append(dict(step=step, **vm))
                fabric.print(f"step {step:5d} | validation loss {vm['val_loss']:.4f} | ppl {vm['val_ppl']:.2f}")
            if step >= total_steps:
                break
    if cfg.save_final_checkpoint and fabric.global_rank == 0:
        path = os.path.join(cfg.out_path, cfg.run_name, "final_checkpoint")
        model.save_pretrained(path)
        fabric.print(f"saved {path}")
    fabric.barrier()
    fabric.shutdown()
    return {"losses": losses, "steps": step, "validations": validations}


def parse(argv=None) -> CLISettings:
    cfg = CLISettings()
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    for key, val in asdict(cfg).items():
        if isinstance(val, dict):
            ap.add_argument(f"--{key}", type=json.loads, default=val)
        elif isinstance(val, bool):
            ap.add_argument(f"--{key}", type=lambda s: s.lower() in ("1", "true", "yes"), default=val)
        else:
            ap.add_argument(f"--{key}", type=type(val) if val is not None else str, default=val)
    ns = vars(ap.parse_args(argv))
    for k in ("max_samples", "num_steps"):
        ns[k] = int(ns[k]) if ns[k] is not None else None
    return CLISettings(**ns)


if __name__ == "__main__":
    train(parse())
