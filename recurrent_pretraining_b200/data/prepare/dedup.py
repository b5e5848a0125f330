"""Near-duplicate and repeated-passage removal on parquet text shards.

Counterparts of scripts/parquet_to_parquet_dedup.py (MinHash signatures -> LSH buckets -> clusters -> keep one per
cluster) and scripts/parquet_to_parquet_sentence_dedup.py (spans of consecutive sentences that already occurred
elsewhere are cut out), which run on datatrove + SLURM in the reference.  Same algorithms, single process, numpy."""
from __future__ import annotations

import hashlib
import re
from typing import Iterable, Sequence

import numpy as np

_MERSENNE = (1 << 61) - 1
_TOKEN = re.compile(r"\w+", re.UNICODE)
_SENT = re.compile(r"(?<=[.!?。！？])\s+|\n+")


def _h64(data: bytes) -> int:
    return int.from_bytes(hashlib.blake2b(data, digest_size=8).digest(), "little")


def shingles(text: str, n: int = 5) -> set:
    words = [w.lower() for w in _TOKEN.findall(text)]
    if len(words) < n:
        return {_h64(" ".join(words).encode())} if words else set()
    return {_h64(" ".join(words[i:i + n]).encode()) for i in range(len(words) - n + 1)}


class MinHasher:
    """``num_buckets * hashes_per_bucket`` permutations ``(a * x + b) mod (2^61 - 1)`` of 64-bit shingle hashes."""

    def __init__(self, num_buckets: int = 14, hashes_per_bucket: int = 8, n_grams: int = 5, seed: int = 1):
        self.nb, self.hb, self.n = num_buckets, hashes_per_bucket, n_grams
        rng = np.random.default_rng(seed)
        k = num_buckets * hashes_per_bucket
        self.a = rng.integers(1, _MERSENNE, size=k, dtype=np.uint64).astype(object)
        self.b = rng.integers(0, _MERSENNE, size=k, dtype=np.uint64).astype(object)

    def signature(self, text: str) -> np.ndarray:
        sh = shingles(text, self.n)
        if not sh:
            return np.full(self.nb * self.hb, _MERSENNE, dtype=np.uint64)
        x = np.array([s % _MERSENNE for s in sh], dtype=object)
        vals = (np.outer(self.a, x) + self.b[:, None]) % _MERSENNE
        return vals.min(axis=1).astype(np.uint64)

    def bucket_keys(self, sig: np.ndarray) -> list:
        return [(i, _h64(sig[i * self.hb:(i + 1) * self.hb].tobytes())) for i in range(self.nb)]


class _UnionFind:
    def __init__(self, n):
        self.p = list(range(n))

    def find(self, x):
        while self.p[x] != x:
            self.p[x] = self.p[self.p[x]]
            x = self.p[x]
        return x

    def union(self, a, b):
        ra, rb = self.find(a), self.find(b)
        if ra != rb:
            self.p[max(ra, rb)] = min(ra, rb)


def minhash_clusters(texts: Sequence[str], hasher: MinHasher | None = None) -> list:
    """Cluster id per document: documents that share at least one LSH bucket end up in the same cluster."""
    hasher = hasher or MinHasher()
    uf = _UnionFind(len(texts))
    seen: dict = {}
    for i, t in enumerate(texts):
        for key in hasher.bucket_keys(hasher.signature(t)):
            j = seen.setdefault(key, i)
            if j != i:
                uf.union(i, j)
    return [uf.find(i) for i in range(len(texts))]


def minhash_dedup(texts: Sequence[str], hasher: MinHasher | None = None) -> list:
    """Indices of the documents to keep (the first member of every near-duplicate cluster)."""
    clusters = minhash_clusters(texts, hasher)
    return [i for i, c in enumerate(clusters) if c == i]


def split_sentences(text: str) -> list:
    return [s for s in _SENT.split(text) if s.strip()]


def sentence_dedup(texts: Iterable[str], span: int = 3, min_doc_words: int = 0) -> list:
    """Cut every run of ``span`` consecutive sentences that already occurred earlier in the stream (in this or another
    document).  Returns the filtered texts (documents that fall under ``min_doc_words`` words become empty strings)."""
    seen: set = set()
    out = []
    for text in texts:
        sents = split_sentences(text)
        drop = [False] * len(sents)
        norm = [" ".join(_TOKEN.findall(s.lower())) for s in sents]
        for i in range(len(sents) - span + 1):
            key = _h64("\x1f".join(norm[i:i + span]).encode())
            if key in seen:
                for j in range(i, i + span):
                    drop[j] = True
            else:
                seen.add(key)
        kept = " ".join(s.strip() for s, d in zip(sents, drop) if not d)
        out.append(kept if len(_TOKEN.findall(kept)) >= min_doc_words else "")
    return out


def dedup_parquet(files: Sequence[str], out_dir: str, column: str = "text", mode: str = "minhash", **kw) -> dict:
    """Read the shards, deduplicate over ALL of them, write one output shard per input shard."""
    import os

    import pyarrow as pa
    import pyarrow.parquet as pq

    os.makedirs(out_dir, exist_ok=True)
    per_file = [pq.read_table(f, columns=[column]).column(column).to_pylist() for f in files]
    flat = [t for rows in per_file for t in rows]
    if mode == "minhash":
        keep = set(minhash_dedup(flat, MinHasher(**kw) if kw else None))
        new = [t if i in keep else None for i, t in enumerate(flat)]
    else:
        new = [t or None for t in sentence_dedup(flat, **kw)]
    pos, written = 0, 0
    for f, rows in zip(files, per_file):
        part = [t for t in new[pos:pos + len(rows)] if t is not None]
        pos += len(rows)
        written += len(part)
        pq.write_table(pa.table({column: part}), os.path.join(out_dir, os.path.basename(f)))
    return {"documents_in": len(flat), "documents_out": written}
