"""Fetch the raw sources of a manifest into local parquet shards.

Counterpart of scripts/scalable_data_download.py, scripts/the_stack_downloader.py and
scripts/download_stream_to_local_copy.py: every source of the manifest (``unify_filter.load_sources``) is streamed from
its address and saved as parquet; rows of code datasets that carry only a Software Heritage blob id get their content
from the public blob store (gzip members under ``content/<blob_id>``), many requests in flight.  There is no network on
the build machines, so the transport is a parameter: ``open_source(source) -> iterable of rows`` and
``fetch_blob(blob_id) -> bytes``; the defaults use ``datasets`` / ``urllib`` when a network exists."""
from __future__ import annotations

import concurrent.futures as cf
import gzip
import os
from typing import Callable, Iterable, Iterator, Optional

from .unify_filter import DataSource, save_as_parquet

BLOB_URL = "https://softwareheritage.s3.amazonaws.com/content/{blob_id}"


def default_open_source(source: DataSource) -> Iterable[dict]:
    import datasets  # needs network access or a populated cache

    ds = datasets.load_dataset(source.address, source.subset, streaming=True)
    for split in ds.values():
        yield from split


def default_fetch_blob(blob_id: str, timeout: float = 30.0) -> bytes:
    import urllib.request

    with urllib.request.urlopen(BLOB_URL.format(blob_id=blob_id), timeout=timeout) as r:
        return r.read()


def decode_blob(raw: bytes, encoding: Optional[str] = None) -> str:
    """Blobs are stored gzip-compressed; the source encoding comes with the row (default utf-8, undecodable bytes are
    replaced)."""
    try:
        raw = gzip.decompress(raw)
    except (OSError, EOFError):
        pass
    return raw.decode(encoding or "utf-8", errors="replace")


def attach_blob_contents(rows: Iterable[dict], fetch_blob: Callable[[str], bytes] = default_fetch_blob,
                         max_workers: int = 32, batch: int = 1024, id_key: str = "blob_id",
                         encoding_key: str = "src_encoding") -> Iterator[dict]:
    """Rows with ``blob_id`` -> rows with ``content``; a failed download yields the row with empty content (and is
    counted in ``row["download_error"]``) rather than stopping a run of millions of files."""
    def one(row):
        try:
            row["content"] = decode_blob(fetch_blob(row[id_key]), row.get(encoding_key))
        except Exception as exc:  # noqa: BLE001
            row["content"], row["download_error"] = "", f"{type(exc).__name__}: {exc}"[:120]
        return row

    chunk = []
    with cf.ThreadPoolExecutor(max_workers=max_workers) as pool:
        for row in rows:
            chunk.append(dict(row))
            if len(chunk) == batch:
                yield from pool.map(one, chunk)
                chunk = []
        if chunk:
            yield from pool.map(one, chunk)


def download_sources(sources: dict, out_dir: str, open_source: Callable = default_open_source,
                     fetch_blob: Callable[[str], bytes] = default_fetch_blob, limit: Optional[int] = None,
                     target_shard_bytes: int = 2 * 1024 ** 3) -> dict:
    """Every source -> ``out_dir/<name>_*.parquet`` with a ``text`` column (first listed feature, or the fetched blob
    content).  Sources whose shards already exist are skipped.  Returns ``{name: [paths]}``."""
    done = {}
    for name, src in sources.items():
        existing = sorted(p for p in (os.listdir(out_dir) if os.path.isdir(out_dir) else [])
                          if p.startswith(name + "_") and p.endswith(".parquet"))
        if existing:
            done[name] = [os.path.join(out_dir, p) for p in existing]
            continue
        rows = open_source(src)
        if src.requires_software_heritage_aws_download:
            rows = attach_blob_contents(rows, fetch_blob)
            key = "content"
        else:
            key = None

        def texts():
            for i, r in enumerate(rows):
                if limit is not None and i >= limit:
                    return
                if key is not None:
                    yield {"text": r[key]}
                elif len(src.features) == 1 and isinstance(r.get(src.features[0]), str):
                    yield {"text": r[src.features[0]]}
                else:
                    from .unify_filter import unify_row

                    yield unify_row(r, src)

        done[name] = save_as_parquet(texts(), out_dir, name, target_shard_bytes, resume=False)
    return done
