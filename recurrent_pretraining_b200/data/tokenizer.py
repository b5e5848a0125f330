"""Thin tokenizer wrapper around a Hugging Face ``tokenizer.json`` directory (recpre/tokenizer.py:10-134).

Discovers bos/eos/pad ids from ``tokenizer_config.json`` / ``generation_config.json``, encodes to int32 tensors with
optional bos/eos, and pickles as its directory path.  A missing directory gives an *uninitialised* tokenizer (special
ids taken from the Huginn vocabulary) so that synthetic-data runs need no tokenizer files.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional, Union

import torch

HUGINN_IDS = {"bos": 65504, "eos": 65505, "end_turn": 65508, "pad": 65509}


class Tokenizer:
    def __init__(self, checkpoint_dir: Union[Path, str, None], allow_missing: bool = True,
                 broken_state_load_fallback: Optional[bool] = None):
        if broken_state_load_fallback is not None:       # the reference's name for the same switch
            allow_missing = bool(broken_state_load_fallback)
        self.checkpoint_dir = Path(checkpoint_dir) if checkpoint_dir else None
        self.processor = None
        self.backend = None
        self.bos_id, self.eos_id, self.pad_id = HUGINN_IDS["bos"], HUGINN_IDS["eos"], HUGINN_IDS["pad"]
        # ids that the cache-attention / document-block options would need; no tokenizer of the reference defines them
        # (recpre/tokenizer.py:33-34), so those options stay off
        self.cache_token_id = self.eod_token_id = None
        if self.checkpoint_dir is None or not self.checkpoint_dir.exists():
            if not allow_missing:
                raise NotADirectoryError(f"Tokenizer checkpoint {checkpoint_dir} cannot be loaded.")
            return
        d = self.checkpoint_dir
        if not (d / "tokenizer.json").is_file():
            raise NotImplementedError("Couldn't load a tokenizer from the given checkpoint directory.")
        from transformers import AutoTokenizer, PreTrainedTokenizerFast

        try:
            self.processor = AutoTokenizer.from_pretrained(str(d), add_bos_token=False, add_eos_token=False)
        except Exception:
            self.processor = PreTrainedTokenizerFast(tokenizer_file=str(d / "tokenizer.json"))
        self.backend = "huggingface"
        self.bos_id = self.processor.bos_token_id
        self.eos_id = self.processor.eos_token_id
        self.pad_id = self.processor.pad_token_id
        gen = d / "generation_config.json"
        if gen.is_file():
            cfg = json.loads(gen.read_text())
            self.bos_id = self.bos_id if self.bos_id is not None else cfg.get("bos_token_id")
            self.eos_id = self.eos_id if self.eos_id is not None else cfg.get("eos_token_id")
            self.pad_id = self.pad_id if self.pad_id is not None else cfg.get("pad_token_id")

    @property
    def vocab_size(self) -> int:
        return self.processor.vocab_size if self.processor is not None else 65536

    def __len__(self) -> int:
        return len(self.processor) if self.processor is not None else 65536

    def encode(self, string: str, device: Optional[torch.device] = None, bos: Optional[bool] = None, eos: bool = False,
               max_length: int = -1) -> torch.Tensor:
        if self.processor is None:
            raise RuntimeError("tokenizer files are not available")
        ids = self.processor.encode(string, add_special_tokens=False)
        if bos:
            if self.bos_id is None:
                raise NotImplementedError("This tokenizer does not have a defined bos token")
            ids = [self.bos_id] + ids
        if eos:
            ids = ids + [self.eos_id]
        if max_length > 0:
            ids = ids[:max_length]
        return torch.tensor(ids, dtype=torch.int, device=device)

    def decode(self, tensor: torch.Tensor, skip_special_tokens: bool = False) -> str:
        ids = [tensor.item()] if tensor.ndim == 0 else tensor.tolist()
        return self.processor.decode(ids, skip_special_tokens=skip_special_tokens)

    def state_dict(self):
        return {"dir": str(self.checkpoint_dir)}

    def load_state_dict(self, state_dict):
        """The tokenizer recorded in a checkpoint, or this one when its folder no longer exists."""
        try:
            return Tokenizer(state_dict["dir"])
        except Exception as exc:  # noqa: BLE001
            print(f"Warning: could not reload the checkpoint's tokenizer ({exc}); keeping the configured one.")
            return self

    def __reduce__(self):
        return (self.__class__, (self.checkpoint_dir,))
