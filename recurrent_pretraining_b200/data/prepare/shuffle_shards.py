"""Reshuffle packed rows across shards in rounds: each round reads a random group of shards, permutes all of their
rows together and writes the group back, so after a few rounds every row can have reached any shard while only one
group is ever held in memory.

Counterpart of scripts/parquet_to_parquet_shuffler.py:150-204.
"""
from __future__ import annotations

import argparse
import glob
import os
import random


def shuffle_round(paths: list, group_size: int, rng: random.Random, row_group_size: int = 1024) -> None:
    import pyarrow as pa
    import pyarrow.parquet as pq

    order = list(paths)
    rng.shuffle(order)
    for g in range(0, len(order), group_size):
        group = order[g:g + group_size]
        tables = [pq.read_table(p) for p in group]
        sizes = [t.num_rows for t in tables]
        merged = pa.concat_tables(tables)
        perm = list(range(merged.num_rows))
        rng.shuffle(perm)
        merged = merged.take(pa.array(perm))
        start = 0
        for p, n in zip(group, sizes):
            tmp = p + ".tmp"
            pq.write_table(merged.slice(start, n), tmp, row_group_size=row_group_size)
            os.replace(tmp, p)  # a crash never leaves a half-written shard under the real name
            start += n


def shuffle_shards(folder: str, rounds: int = 3, group_size: int = 16, seed: int = 4242, prefix: str = "") -> int:
    paths = sorted(glob.glob(os.path.join(folder, f"{prefix}*.parquet")))
    rng = random.Random(seed)
    for _ in range(rounds):
        shuffle_round(paths, group_size, rng)
    return len(paths)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("folder")
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--group_size", type=int, default=16)
    ap.add_argument("--seed", type=int, default=4242)
    a = ap.parse_args(argv)
    print(f"shuffled {shuffle_shards(a.folder, a.rounds, a.group_size, a.seed)} shards")


if __name__ == "__main__":
    main()
