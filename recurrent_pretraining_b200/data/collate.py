"""Batch assembly: shift-by-one inputs/labels, optional on-the-fly tokenisation of text rows.

Contract (recpre/data_loading_utils.py:102-205): rows of ``block_size + 1`` ids give ``input = row[:, :-1]`` and
``labels = row[:, 1:]`` (int64); pad ids in the *inputs* are replaced by eos; an all-padding batch ends the epoch.
Text rows are dicts carrying a ``data_signature`` whose ``format_fn`` names how fields become (tokens, labels).
"""
from __future__ import annotations

from typing import Optional

import torch


def pass_text(row, tok, add_bos, add_eos):
    ids = tok.encode(row["text"], bos=add_bos, eos=add_eos)
    return ids, ids.clone()


def concat_input_target(row, tok, add_bos, add_eos):
    ids = tok.encode(row["input"] + row["target"], bos=add_bos, eos=add_eos)
    return ids, ids.clone()


def condition_input_supervise_target(row, tok, add_bos, add_eos):
    prompt = tok.encode(row["input"], bos=add_bos, eos=False)
    joint = tok.encode(row["input"] + row["target"], bos=add_bos, eos=add_eos)
    labels = joint.clone()
    labels[: len(prompt)] = tok.pad_id
    return joint, labels


def chat_supervise_all(row, tok, add_bos, add_eos):
    key = row["data_signature"]["keys"][0]
    text = tok.processor.apply_chat_template(row[key], tokenize=False)
    ids = tok.encode(text, bos=add_bos, eos=add_eos)
    return ids, ids.clone()


def chat_supervise_assistant(row, tok, add_bos, add_eos):
    key = row["data_signature"]["keys"][0]
    enc = tok.processor.apply_chat_template(row[key], tokenize=True, add_generation_prompt=False,
                                            return_assistant_tokens_mask=True, return_dict=True, return_tensors="pt")
    ids = enc["input_ids"][0]
    mask = torch.as_tensor(enc["assistant_masks"]).reshape(-1).bool()
    labels = torch.where(mask, ids, torch.full_like(ids, tok.pad_id))
    return ids, labels


apply_chat_template_supervise_all = chat_supervise_all                 # the reference's function names
apply_chat_template_supervise_assistant = chat_supervise_assistant

FORMAT_FNS = {
    "pass_text": pass_text,
    "concat_input_target": concat_input_target,
    "condition_input_supervise_target": condition_input_supervise_target,
    "apply_chat_template_supervise_all": chat_supervise_all,
    "apply_chat_template_supervise_assistant": chat_supervise_assistant,
}


def apply_formatting(row, tok, add_bos, add_eos):
    if isinstance(row, torch.Tensor):
        return row, row.clone()
    if isinstance(row, dict):
        if "input_ids" in row and "data_signature" not in row:
            t = torch.as_tensor(row["input_ids"])
            return t, t.clone()
        sig = row["data_signature"]
        add_bos = sig.get("add_bos", add_bos) if sig.get("add_bos") is not None else add_bos
        add_eos = sig.get("add_eos", add_eos) if sig.get("add_eos") is not None else add_eos
        return FORMAT_FNS[sig["format_fn"]](row, tok, add_bos, add_eos)
    raise ValueError("Row format not recognized.")


def shift_inputs_and_labels(inputs: torch.Tensor, labels: torch.Tensor, pad_id=None, eos_id=None):
    x = inputs[:, :-1].contiguous().long()
    y = labels[:, 1:].contiguous().long()
    if eos_id is not None and pad_id is not None:
        x[x == pad_id] = eos_id
    return x, y


def generic_collate_fn(batch, tokenizer=None, block_size: Optional[int] = None, pad_to_block_size: bool = False,
                       add_bos: bool = True, add_eos: bool = True, collate_checks_enabled: bool = True,
                       all_block_size_tensors: bool = False):
    pad_id = getattr(tokenizer, "pad_id", None)
    eos_id = getattr(tokenizer, "eos_id", None)
    metadata = [row.get("data_id") if isinstance(row, dict) else None for row in batch]
    if all_block_size_tensors:
        rows = [r["input_ids"] if isinstance(r, dict) else r for r in batch]
        stacked = torch.stack(rows)
        x, y = shift_inputs_and_labels(stacked, stacked.clone(), pad_id, eos_id)
        return x, y, metadata
    if block_size is None:
        raise ValueError("block_size is required unless all_block_size_tensors is set")
    if collate_checks_enabled:
        if not isinstance(batch, list) or not all(isinstance(r, (dict, torch.Tensor)) for r in batch):
            raise TypeError("Batch must be a list of dicts or tensors.")
        if any(isinstance(r, dict) and "data_signature" in r for r in batch):
            if tokenizer is None or pad_id is None:
                raise ValueError("Text rows need a tokenizer with a pad id.")
    pairs = [apply_formatting(r, tokenizer, add_bos, add_eos) for r in batch]
    width = block_size if pad_to_block_size else min(max(len(t) for p in pairs for t in p), block_size)
    fill = pad_id or 0
    inputs = torch.full((len(pairs), width), fill, dtype=torch.int)
    labels = torch.full((len(pairs), width), fill, dtype=torch.int)
    for i, (a, b) in enumerate(pairs):
        inputs[i, : min(len(a), width)] = a[:width]
        labels[i, : min(len(b), width)] = b[:width]
    if (eos_id is not None and bool(torch.all(labels == eos_id))) or (pad_id is not None and bool(torch.all(labels == pad_id))):
        raise StopIteration("All tokens in batch are padding tokens.")
    x, y = shift_inputs_and_labels(inputs, labels, pad_id, eos_id)
    return x, y, metadata
