"""Raw text -> training shards: tokenise every document (bos ... eos), shuffle the documents globally, pack the token
stream into rows of ``block_size + 1`` tokens, write ``num_shards`` parquet files with one ``input_ids`` column, and
split them into train / validation folders.

Counterpart of scripts/parquet_to_parquet_tokenizer.py:227-399.  The row length is block_size + 1 because the collate
function shifts inputs and labels by one (data contract: a row of 4097 tokens yields 4096 inputs and 4096 labels).
A document tail that does not fill a row is dropped ("incinerated") unless ``every_token_is_sacred``, in which case it
is carried over into the next row.

    python -m recurrent_pretraining_b200.data.prepare.tokenize_pack --files raw/*.parquet --tokenizer tok/ --out data/
"""
from __future__ import annotations

import argparse
import glob
import os
import random

import numpy as np

from .tokenizer_train import iter_texts


def tokenize_documents(texts, encode, bos_id: int, eos_id: int):
    for t in texts:
        ids = encode(t)
        if len(ids):
            yield np.asarray([bos_id, *ids, eos_id], dtype=np.int32)


def pack_rows(docs, row_len: int, every_token_is_sacred: bool = False):
    """Documents are laid end to end and rows are cut every ``row_len`` tokens.  The unfinished remainder at the end of
    the stream is dropped, or, with ``every_token_is_sacred``, completed with copies of its last token (an eos)."""
    buf = np.empty(0, dtype=np.int32)
    for d in docs:
        buf = np.concatenate([buf, d])
        while len(buf) >= row_len:
            yield buf[:row_len]
            buf = buf[row_len:]
    if every_token_is_sacred and len(buf):
        pad = np.full(row_len - len(buf), buf[-1], dtype=np.int32)  # repeat eos: labels there are real eos tokens
        yield np.concatenate([buf, pad])


def write_shards(rows: list, out_dir: str, num_shards: int, prefix: str, row_group_size: int = 1024) -> list:
    import pyarrow as pa
    import pyarrow.parquet as pq

    os.makedirs(out_dir, exist_ok=True)
    paths = []
    for s in range(num_shards):
        part = rows[s::num_shards]
        if not part:
            continue
        table = pa.table({"input_ids": pa.array([r.tolist() for r in part], type=pa.list_(pa.int32()))})
        path = os.path.join(out_dir, f"{prefix}_{s:05d}.parquet")
        pq.write_table(table, path, row_group_size=row_group_size)
        paths.append(path)
    return paths


def prepare(files, encode, bos_id: int, eos_id: int, out_dir: str, block_size: int = 4096, num_shards: int = 8,
            val_fraction: float = 0.05, seed: int = 1337, every_token_is_sacred: bool = False, column: str = "text",
            row_group_size: int = 1024) -> dict:
    docs = list(tokenize_documents(iter_texts(files, column), encode, bos_id, eos_id))
    rng = random.Random(seed)
    rng.shuffle(docs)                                           # global document shuffle before packing
    rows = list(pack_rows(docs, block_size + 1, every_token_is_sacred))
    rng.shuffle(rows)                                           # and a row shuffle before sharding
    n_val = max(1, int(len(rows) * val_fraction)) if len(rows) > 1 and val_fraction > 0 else 0
    val, train = rows[:n_val], rows[n_val:]
    info = {"documents": len(docs), "tokens": int(sum(len(d) for d in docs)), "rows": len(rows),
            "train": write_shards(train, os.path.join(out_dir, "train"), num_shards, "train", row_group_size),
            "val": write_shards(val, os.path.join(out_dir, "val"), max(1, num_shards // 8), "val", row_group_size)}
    info["dropped_tokens"] = info["tokens"] - len(rows) * (block_size + 1) if not every_token_is_sacred else 0
    return info


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--files", nargs="+", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--block_size", type=int, default=4096)
    ap.add_argument("--num_shards", type=int, default=4096)
    ap.add_argument("--val_fraction", type=float, default=0.05)
    ap.add_argument("--seed", type=int, default=1337)
    ap.add_argument("--every_token_is_sacred", action="store_true")
    ap.add_argument("--column", default="text")
    a = ap.parse_args(argv)
    from ..tokenizer import Tokenizer

    tok = Tokenizer(a.tokenizer)
    files = [f for pat in a.files for f in sorted(glob.glob(pat))]
    info = prepare(files, lambda s: tok.encode(s, bos=False, eos=False).tolist(), tok.bos_id, tok.eos_id, a.out,
                   a.block_size, a.num_shards, a.val_fraction, a.seed, a.every_token_is_sacred, a.column)
    print({k: (len(v) if isinstance(v, list) else v) for k, v in info.items()})


if __name__ == "__main__":
    main()
