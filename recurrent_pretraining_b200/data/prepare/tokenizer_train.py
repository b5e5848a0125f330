"""Train a byte-level BPE tokenizer whose special tokens sit at the end of the vocabulary.

Counterpart of scripts/tokenizer_generation.py:427-748 (which trains with the `bpeasy` package and a long hand-tuned
pre-tokenisation regex).  `bpeasy` is not available here; this uses the `tokenizers` library with a compact
pre-tokenisation pattern built for the same goals: digits split one by one, runs of newlines kept together, LaTeX
commands and code operators kept whole, at most one leading space attached to a word.

    python -m recurrent_pretraining_b200.data.prepare.tokenizer_train --files corpus/*.txt --vocab_size 65536 --out tok/
"""
from __future__ import annotations

import argparse
import glob
import json
import os

from .special_tokens import N_SPECIAL, SPECIAL_TOKENS, special_token_ids

PRETOKENIZE = (r"\\[a-zA-Z]+|\n+|\p{N}|==|!=|<=|>=|\*\*|//|->|=>|::|\+=|-=|"
               r" ?\p{L}+(?:['’]\p{L}+)?| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+")


EMOJI_RANGES = ((0x1F600, 0x1F64F), (0x1F300, 0x1F5FF), (0x1F680, 0x1F6FF), (0x1F900, 0x1F9FF), (0x2600, 0x26FF))
MATH_RANGES = ((0x2200, 0x22FF), (0x27C0, 0x27EF), (0x2980, 0x29FF), (0x2A00, 0x2AFF), (0x2190, 0x21FF),
               (0x0391, 0x03C9), (0x2070, 0x209F))


def manual_tokens() -> list:
    """Tokens put into the vocabulary by hand before BPE fills the rest (scripts/tokenizer_generation.py:599-611):
    quote runs used by code, runs of 1..16 spaces / newlines / tabs, the first 687 code points (Latin + IPA) so that
    basic text never falls back to bytes, emoji and mathematical symbol blocks, and the assistant's name."""
    out = ['"' * 3, "'" * 3, '"', "'" * 2, 'f"', "f'"]
    for ch in (" ", "\n", "\t"):
        out += [ch * n for n in range(1, 17)]
    out += [chr(i) for i in range(687)]
    out += [chr(0x1F9AD)]
    for lo, hi in EMOJI_RANGES + MATH_RANGES:
        out += [chr(i) for i in range(lo, hi + 1)]
    out.append("Huginn")
    seen, uniq = set(), []
    for t in out:
        if t not in seen and t:
            seen.add(t)
            uniq.append(t)
    return uniq


def iter_texts(files, column: str = "text"):
    for f in files:
        if f.endswith(".parquet"):
            import pyarrow.parquet as pq

            pf = pq.ParquetFile(f)
            for g in range(pf.num_row_groups):
                yield from pf.read_row_group(g, columns=[column]).column(column).to_pylist()
        elif f.endswith(".jsonl"):
            with open(f) as fh:
                for line in fh:
                    yield json.loads(line)[column]
        else:
            with open(f, errors="replace") as fh:
                yield fh.read()


def train_tokenizer(files, vocab_size: int = 65536, out_dir: str = "tokenizer", column: str = "text",
                    min_frequency: int = 2, add_manual_tokens: bool = False):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers

    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(PRETOKENIZE), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    manual = manual_tokens() if add_manual_tokens else []
    trainer = trainers.BpeTrainer(vocab_size=vocab_size - N_SPECIAL - len(manual), min_frequency=min_frequency,
                                  show_progress=False, initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(iter_texts(files, column), trainer=trainer)
    if manual:
        tok.add_tokens([t for t in manual if tok.token_to_id(t) is None])
    # pad the learned vocabulary so that the specials land on the last N_SPECIAL ids even for a tiny corpus
    missing = (vocab_size - N_SPECIAL) - tok.get_vocab_size()
    if missing > 0:
        tok.add_tokens([f"<|unused_{i}|>" for i in range(missing)])
    tok.add_special_tokens(SPECIAL_TOKENS + [f"<|reserved_{i}|>" for i in range(N_SPECIAL - len(SPECIAL_TOKENS))])
    os.makedirs(out_dir, exist_ok=True)
    tok.save(os.path.join(out_dir, "tokenizer.json"))
    ids = special_token_ids(vocab_size)
    with open(os.path.join(out_dir, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "bos_token": "<|begin_text|>",
                   "eos_token": "<|end_text|>", "pad_token": "<|pad|>", "model_max_length": 4096,
                   "special_token_ids": ids}, f, indent=1)
    return tok


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--files", nargs="+", required=True)
    ap.add_argument("--vocab_size", type=int, default=65536)
    ap.add_argument("--out", default="tokenizer")
    ap.add_argument("--column", default="text")
    ap.add_argument("--manual_tokens", action="store_true", help="reserve the hand-picked tokens (see manual_tokens)")
    a = ap.parse_args(argv)
    files = [f for pat in a.files for f in sorted(glob.glob(pat))]
    tok = train_tokenizer(files, a.vocab_size, a.out, a.column, add_manual_tokens=a.manual_tokens)
    print(f"vocab {tok.get_vocab_size()} -> {a.out}")


if __name__ == "__main__":
    main()
