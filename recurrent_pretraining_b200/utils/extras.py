"""Small utilities that the reference keeps in recpre/utils.py besides the fabric: a streaming checkpoint writer
(``incremental_save``, recpre/utils.py:112-257), exact-match memorisation metrics (``:263-486``), a chunked cross entropy
(``:536-597``) and napkin FLOP estimates (``:639-727``).  Restated here with the same inputs and results; none of them
is on a hot path."""
from __future__ import annotations

import io
import json
import zipfile
from typing import Optional, Sequence

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------------
# streaming checkpoint writer
# ------------------------------------------------------------------------------------------------------
class incremental_save:  # noqa: N801  (kept as the reference's name)
    """Write a (large) state dict one tensor at a time, so that never more than one tensor sits in host memory:

        with incremental_save(path) as saver:
            for name, tensor in model.state_dict().items():
                saver.store(name, tensor)          # moved to the CPU, written, released
            saver.store_meta({"step": 10})

    The file is an uncompressed zip: ``index.json`` (dtype, shape, member name per tensor, plus the metadata) and one
    raw little-endian member per tensor.  ``load_incremental`` reads it back, optionally only some names."""

    def __init__(self, path: str):
        self.path, self.index, self.meta = str(path), {}, {}
        self.zf: Optional[zipfile.ZipFile] = None

    def __enter__(self):
        self.zf = zipfile.ZipFile(self.path + ".tmp", "w", compression=zipfile.ZIP_STORED, allowZip64=True)
        return self

    def store(self, name: str, tensor: torch.Tensor) -> None:
        t = tensor.detach().to("cpu").contiguous()
        member = f"t{len(self.index):06d}.bin"
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        self.zf.writestr(member, raw)
        self.index[name] = {"dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape), "member": member}

    def store_meta(self, meta: dict) -> None:
        self.meta.update(meta)

    def __exit__(self, exc_type, exc, tb):
        import os

        if exc_type is None:
            self.zf.writestr("index.json", json.dumps({"tensors": self.index, "meta": self.meta}))
        self.zf.close()
        if exc_type is None:
            os.replace(self.path + ".tmp", self.path)
        else:
            os.remove(self.path + ".tmp")
        return False


def load_incremental(path: str, names: Optional[Sequence[str]] = None) -> tuple[dict, dict]:
    """(tensors, meta) of a file written by ``incremental_save``."""
    out = {}
    with zipfile.ZipFile(path) as zf:
        idx = json.loads(zf.read("index.json"))
        for name, e in idx["tensors"].items():
            if names is not None and name not in names:
                continue
            dtype = getattr(torch, e["dtype"])
            raw = bytearray(zf.read(e["member"]))
            t = torch.frombuffer(raw, dtype=torch.uint8).view(dtype) if raw else torch.empty(0, dtype=dtype)
            out[name] = t.reshape(e["shape"]).clone()
    return out, idx["meta"]


# ------------------------------------------------------------------------------------------------------
# memorisation (exact match) metrics
# ------------------------------------------------------------------------------------------------------
@torch.no_grad()
def batch_exact_match(logits: torch.Tensor, labels: torch.Tensor, metadata: Sequence, prefix_lengths: Sequence[int],
                      suffix_lengths: Sequence[int], pad_id: int) -> dict:
    """For every row: would greedy decoding have reproduced ``suffix`` tokens after ``prefix`` tokens?  The test is
    teacher-forced: all positions prefix .. prefix+suffix-1 must be argmax-correct.  Returns
    ``{prefix: {suffix: [(hit, metadata_row), ...]}}`` plus the key ``"natural_suffix"`` (the last ``suffix`` tokens of
    the row, and ``"unmasked"``: every non-pad position).  Rows whose padding is not only at the tail contribute to
    ``"unmasked"`` alone."""
    stats = {pl: {sl: [] for sl in suffix_lengths} for pl in prefix_lengths}
    stats["natural_suffix"] = {sl: [] for sl in suffix_lengths}
    stats["natural_suffix"]["unmasked"] = []
    correct = logits.argmax(-1) == labels
    for ok, lab, meta in zip(correct, labels, metadata):
        valid = lab != pad_id
        n = int(valid.sum())
        if bool(valid[:n].all()):            # padding only at the end
            row = ok[:n]
            for pl in prefix_lengths:
                for sl in suffix_lengths:
                    if pl + sl <= n:
                        stats[pl][sl].append((bool(row[pl:pl + sl].all()), meta))
            for sl in suffix_lengths:
                if sl <= n:
                    stats["natural_suffix"][sl].append((bool(row[n - sl:].all()), meta))
        stats["natural_suffix"]["unmasked"].append((bool(ok[valid].all()), meta))
    return stats


def reduce_memorization_metrics(stats_list: Sequence[dict], fabric=None, dataset_names: Sequence = ()) -> dict:
    """Hit rates over all batches and ranks: ``{"em/<prefix>/<suffix>": rate, ...}`` and, for every name in
    ``dataset_names`` that appears as a row's metadata, ``"em/<name>/<prefix>/<suffix>"``."""
    keys, table = [], {}
    for stats in stats_list:
        for pl, inner in stats.items():
            for sl, rows in inner.items():
                for hit, meta in rows:
                    for key in ([f"em/{pl}/{sl}"] + ([f"em/{meta}/{pl}/{sl}"] if meta in dataset_names else [])):
                        h, n = table.get(key, (0, 0))
                        table[key] = (h + int(hit), n + 1)
    keys = sorted(table)
    if fabric is not None and fabric.is_distributed:
        import torch.distributed as dist

        all_keys = [None] * fabric.world_size
        dist.all_gather_object(all_keys, keys)
        keys = sorted(set().union(*all_keys))
    counts = torch.tensor([[table.get(k, (0, 0))[0], table.get(k, (0, 0))[1]] for k in keys], dtype=torch.float64)
    if fabric is not None and fabric.is_distributed and len(keys):
        counts = fabric.all_reduce(counts.to(fabric.device), "sum").cpu()
    return {k: (float(h / n) if n > 0 else float("nan")) for k, (h, n) in zip(keys, counts.tolist())}


# ------------------------------------------------------------------------------------------------------
# chunked cross entropy
# ------------------------------------------------------------------------------------------------------
def chunked_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, chunk_size: int = 128,
                          ignore_indices: Sequence[Optional[int]] = (-1,), reduction: Optional[str] = None,
                          training: bool = True, z_loss_eps: float = 0.0,
                          target_range: Optional[Sequence[int]] = None, return_logits_targets: bool = False):
    """Mean cross entropy over non-ignored positions, evaluated ``chunk_size`` rows at a time so that the softmax
    temporaries of the whole [tokens, vocab] matrix never exist at once (recpre/utils.py:536-597).  The first entry of
    ``ignore_indices`` is the ignore value (a zero or None there means -100), further entries are folded into it;
    ``target_range`` is a sorted list of vocabulary ids to which the classification is restricted (logits keep those
    columns, the i-th id becomes class i); optional z-loss ``eps * mean(logsumexp^2)`` in training.  With
    ``return_logits_targets`` the logits and targets of the non-ignored rows are returned beside the loss."""
    ignore = ignore_indices[0] or -100
    targets = targets.clone()
    for extra in list(ignore_indices)[1:]:
        if extra is not None and extra != ignore:
            targets[targets == extra] = ignore
    logits = logits.reshape(-1, logits.size(-1))
    targets = targets.reshape(-1)
    if target_range is not None:
        from .helpers import slice_logits_remap_labels

        logits, targets = slice_logits_remap_labels(logits, targets, target_range, list(ignore_indices))
    if chunk_size == 0:
        loss = F.cross_entropy(logits, targets, ignore_index=ignore, **({"reduction": reduction} if reduction else {}))
    else:
        total = logits.new_zeros(())
        for lg, tg in zip(logits.split(chunk_size), targets.split(chunk_size)):
            total = total + F.cross_entropy(lg, tg, ignore_index=ignore, reduction="sum")
        loss = total / (targets != ignore).sum().clamp(min=1)
    if z_loss_eps > 0.0 and training:
        loss = loss + z_loss_eps * torch.logsumexp(logits, dim=-1).pow(2).mean()
    if not return_logits_targets:
        return loss
    keep = targets != ignore
    return loss, logits[keep, :], targets[keep]


# ------------------------------------------------------------------------------------------------------
# napkin FLOP estimates
# ------------------------------------------------------------------------------------------------------
def flops_per_param(max_seq_length: int, n_layer: int, n_embd: int, n_params: int) -> int:
    """2 FLOPs per parameter and token, plus the attention score / value products."""
    return 2 * n_params * max_seq_length + n_layer * 4 * n_embd * max_seq_length ** 2


def estimate_flops(model, training: bool) -> int:
    """Parameter-count estimate of one sequence: trainable parameters cost forward + input-gradient + weight-gradient
    passes, frozen ones forward + input-gradient."""
    train_p = sum(p.numel() for p in model.parameters() if p.requires_grad)
    frozen_p = sum(p.numel() for p in model.parameters() if not p.requires_grad)
    cfg = model.config
    L, E, S = cfg.n_layer, cfg.n_embd, model.max_seq_length
    return (3 if training else 1) * flops_per_param(S, L, E, train_p) + \
        (2 if training else 1) * flops_per_param(S, L, E, frozen_p)


def gptneox_tflops(seconds_per_step: float, world_size: int, batch_size: int, seq_len: int, n_layer: int, n_embd: int,
                   vocab_size: int, checkpointing: bool) -> float:
    """TFLOP/s per device by the GPT-NeoX formula (24 B S L E^2 (1 + S / 6E + V / 16LE), x3 or x4 with recomputation)."""
    f = 24 * (4 if checkpointing else 3) * batch_size * seq_len * n_layer * n_embd ** 2 * \
        (1.0 + seq_len / (6.0 * n_embd) + vocab_size / (16.0 * n_layer * n_embd))
    return f / (seconds_per_step * world_size) / 1e12


def gated_mlp_tflops(seconds_per_step: float, world_size: int, batch_size: int, seq_len: int, n_layer: int, n_embd: int,
                     intermediate: int, vocab_size: int, checkpointing: bool, gated: bool = True) -> float:
    """The Megatron-style count with a (gated) MLP of width ``intermediate``: linear 32 B S E^2 + (24 | 16) B S E I per
    layer, attention 16 B S^2 E per layer, head 6 B S E V; without recomputation the layer terms are scaled by 3/4."""
    B, S, E, I, V, L = batch_size, seq_len, n_embd, intermediate, vocab_size, n_layer
    lin = L * (32 * B * S * E * E + (24 if gated else 16) * B * S * E * I)
    att = L * 16 * B * S * S * E
    head = 6 * B * S * E * V
    f = lin + att + head if checkpointing else 0.75 * (lin + att) + head
    return f / 1e12 / seconds_per_step / world_size
