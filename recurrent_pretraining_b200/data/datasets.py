"""Token sources.  All yield 1-D int64 tensors of ``block_size + 1`` token ids (or dicts for text rows).

* ``RandomTokens``  -- synthetic uniform ids (the ``rngds`` debug source of recpre/huggingface_dataset.py:484-507,
  generated lazily per row instead of as a 10^6-row table).
* ``ParquetStream`` -- pyarrow-only stateful stream over pre-tokenised parquet shards with the sharding, shuffling
  and resume semantics of the reference's production loader (recpre/huggingface_dataset.py:124-294): files are
  globbed on rank 0 and broadcast, shuffled with a seeded RNG, assigned ``rank::max(8, world)``; one row group at a
  time is read, shuffled with a per-dataset ``random.Random`` and popped from the end; the state (file index, row
  group, rows left, RNG state, fingerprint) is all-gathered on save and reloaded modulo the saved world size.
* ``TextRows``      -- (alias ``HuggingfaceDataset``) rows of a list of dicts, a parquet / jsonl file or a
  ``datasets.load_from_disk`` directory, dealt out row by row over ranks x loader workers (tokenised in collate).
"""
from __future__ import annotations

import hashlib
import random
from pathlib import Path

import torch
import torch.distributed as dist
from torch.utils.data import IterableDataset


class RandomTokens(IterableDataset):
    def __init__(self, vocab_size: int = 1024, block_size: int = 4096, seed: int = 233, process_rank: int = 0,
                 length: int = 10**6):
        self.vocab_size, self.block_size, self.seed, self.rank, self.length = vocab_size, block_size, seed, process_rank, length
        self._pos = 0

    def __iter__(self):
        while self._pos < self.length:
            g = torch.Generator().manual_seed(self.seed + 7919 * self.rank + self._pos)
            self._pos += 1
            yield torch.randint(0, self.vocab_size, (self.block_size,), generator=g, dtype=torch.int64)

    def state_dict(self):
        return {"pos": self._pos}

    def load_state_dict(self, sd, **_):
        self._pos = int(sd["pos"])

    load_local_state = load_state_dict


class ParquetStream(IterableDataset):
    def __init__(self, dataset_folder_path: str = "", seed: int = 12345, shuffle: bool = True, num_processes: int = 1,
                 process_rank: int = 0, prefix: str = "", shuffle_filenames: bool = True, column: str = "input_ids",
                 broadcast_glob: bool = True, stateful: bool = True, plan_for_later_rank_expansion_to: int = 8,
                 return_data_id: bool = False, data_id=None, verbose: bool = False, data_signature: dict | None = None,
                 repetitions=None):
        # ``data_signature`` ({"keys": [column]}), ``repetitions`` and ``verbose`` are the reference's argument names
        # (recpre/huggingface_dataset.py:128-145); as there, the token streams do not repeat
        if data_signature is not None and data_signature.get("keys"):
            column = data_signature["keys"][0]
        files = None
        distributed = dist.is_available() and dist.is_initialized()
        if not (broadcast_glob and distributed) or process_rank == 0:
            files = sorted(str(p) for p in Path(dataset_folder_path).glob(f"{prefix}*.parquet"))
        if broadcast_glob and distributed:
            box = [files]
            dist.broadcast_object_list(box, 0)
            files = box[0]
        if shuffle_filenames:
            random.Random(seed).shuffle(files)
        stride = max(plan_for_later_rank_expansion_to, num_processes) if plan_for_later_rank_expansion_to > 0 \
            else num_processes
        self.parquet_files = files[process_rank::stride] if stride > 1 else files
        if not self.parquet_files:
            raise ValueError(f"Empty dataset on rank {process_rank}")
        self.fingerprint = hashlib.shake_128(str(self.parquet_files).encode()).hexdigest(4)
        self.shuffle, self.seed, self.rank, self.stateful, self.column = shuffle, seed, process_rank, stateful, column
        self.return_data_id, self.data_id = return_data_id, data_id
        self._reset()

    def _reset(self):
        self._rng = random.Random(self.seed)
        self._rng_state = None
        self._buffer: list = []
        self._file_idx = 0
        self._row_group_idx = 0

    def _read_buffer(self, pf):
        self._buffer = pf.read_row_group(self._row_group_idx).column(self.column).to_pylist()
        if self.shuffle:
            self._rng_state = self._rng.getstate()
            self._rng.shuffle(self._buffer)

    def __iter__(self):
        import pyarrow.parquet as pq

        if not self.stateful:
            self._reset()
        while self._file_idx < len(self.parquet_files):
            if not self._buffer:
                pf = pq.ParquetFile(self.parquet_files[self._file_idx])
                if self._row_group_idx >= pf.num_row_groups:
                    self._file_idx += 1
                    self._row_group_idx = 0
                    continue
                self._read_buffer(pf)
                self._row_group_idx += 1
            while self._buffer:
                row = torch.as_tensor(self._buffer.pop(), dtype=torch.long)
                yield {"input_ids": row, "data_id": self.data_id} if self.return_data_id else row

    # -- state ---------------------------------------------------------------------------------
    def local_state(self) -> dict:
        return {"file_idx": self._file_idx, "row_group_idx": self._row_group_idx - 1, "row_idx": len(self._buffer),
                "fingerprint": self.fingerprint, "rng_state": self._rng_state}

    def state_dict(self) -> dict:
        return self.state_from_local(self.local_state())

    def load_local_state(self, local: dict) -> None:
        self.load_state_dict({k: [v] for k, v in local.items()}, _rank=0)

    def state_from_local(self, local: dict) -> dict:
        """Per-rank states gathered into lists indexed by rank (a different world size can reload them).  Collective."""
        if dist.is_available() and dist.is_initialized():
            states = [None] * dist.get_world_size()
            dist.all_gather_object(states, local)
        else:
            states = [local]
        return {k: [s[k] for s in states] for k in local}

    def load_state_dict(self, sd: dict, offset_ranks: bool = False, _rank=None) -> None:
        import pyarrow.parquet as pq

        rank = _rank if _rank is not None else (dist.get_rank() if dist.is_available() and dist.is_initialized() else 0)
        pick = lambda key: sd[key][rank % len(sd["fingerprint"])]  # noqa: E731
        if pick("fingerprint") != self.fingerprint:
            print(f"WARNING dataset fingerprint mismatch: expected {self.fingerprint}, got {pick('fingerprint')}")
            self._file_idx, self._row_group_idx, row_idx = 0, 0, 0
        else:
            self._file_idx = max(pick("file_idx"), 0)
            self._row_group_idx = max(pick("row_group_idx"), 0)
            row_idx = max(pick("row_idx"), 0) + (rank % 1000 if offset_ranks else 0)
        state = pick("rng_state")
        if state is not None:
            self._rng = random.Random()
            self._rng.setstate(tuple(state) if not isinstance(state, tuple) else state)
        if pick("row_group_idx") < 0 and pick("fingerprint") == self.fingerprint:
            self._buffer, self._row_group_idx = [], 0     # saved before the first row group was read
            return
        self._read_buffer(pq.ParquetFile(self.parquet_files[self._file_idx]))
        self._buffer = self._buffer[:row_idx]
        self._row_group_idx += 1


class BufferShuffledParquet(IterableDataset):
    """The ``pqds`` source: a plain stream over parquet shards (files ``rank::world``) with a shuffle buffer
    (recpre/huggingface_dataset.py:34-121, which uses HF ``datasets`` streaming with ``shuffle(buffer_size=1024)``).
    Here the buffer is filled with the next ``buffer_size`` rows, shuffled with a seeded RNG and drained, which keeps the
    position resumable exactly: the state is (file, record batch, rows emitted from the current buffer, RNG state at the
    fill), so a resume re-reads one buffer and skips what was already emitted."""

    def __init__(self, dataset_folder_path: str = "", seed: int = 12345, shuffle: bool = True, num_processes: int = 1,
                 process_rank: int = 0, prefix: str = "", shuffle_filenames: bool = True, column: str = "input_ids",
                 buffer_size: int = 1024, read_batch: int = 256, return_data_id: bool = False, data_id=None,
                 broadcast_glob: bool = True, data_signature: dict | None = None, repetitions=None,
                 verbose: bool = True, stateful: bool = True):
        if data_signature is not None and data_signature.get("keys"):     # the reference's name for the column choice
            column = data_signature["keys"][0]
        files = None
        distributed = dist.is_available() and dist.is_initialized()
        if not (broadcast_glob and distributed) or process_rank == 0:
            files = sorted(str(p) for p in Path(dataset_folder_path).glob(f"{prefix}*.parquet"))
            if shuffle_filenames:
                random.Random(seed).shuffle(files)
        if broadcast_glob and distributed:
            box = [files]
            dist.broadcast_object_list(box, 0)
            files = box[0]
        if not files:
            raise FileNotFoundError(f"No files found at {dataset_folder_path} with prefix {prefix}.")
        self.parquet_files = files[process_rank::num_processes] if num_processes > 1 else files
        if not self.parquet_files:
            raise ValueError(f"Empty dataset on rank {process_rank}")
        self.fingerprint = hashlib.shake_128(str(self.parquet_files).encode()).hexdigest(4)
        self.shuffle, self.column, self.buffer_size, self.read_batch = shuffle, column, buffer_size, read_batch
        self.return_data_id, self.data_id = return_data_id, data_id
        self._rng = random.Random(seed)
        self._start = (0, 0)          # (file index, record batch index) where the current buffer starts
        self._emitted = 0             # rows of the current buffer already handed out
        self._fill_rng = self._rng.getstate()

    def _rows_from(self, file_idx: int, batch_idx: int):
        """Yield (row, (file index, next record batch index)) from a position on."""
        import pyarrow.parquet as pq

        for fi in range(file_idx, len(self.parquet_files)):
            pf = pq.ParquetFile(self.parquet_files[fi])
            for bi, rb in enumerate(pf.iter_batches(batch_size=self.read_batch, columns=[self.column],
                                                     use_threads=False)):
                if fi == file_idx and bi < batch_idx:
                    continue
                rows = rb.column(0).to_pylist()
                for j, r in enumerate(rows):
                    last = j == len(rows) - 1
                    yield r, ((fi, bi + 1) if last else None)

    def __iter__(self):
        skip = self._emitted
        while True:
            self._rng.setstate(self._fill_rng)
            buf, nxt = [], None
            for r, boundary in self._rows_from(*self._start):
                buf.append(r)
                if boundary is not None and len(buf) >= self.buffer_size:
                    nxt = boundary        # buffers end on record-batch boundaries, so a position is (file, batch)
                    break
            if not buf:
                return
            if self.shuffle:
                self._rng.shuffle(buf)
            after_rng = self._rng.getstate()
            for i in range(skip, len(buf)):
                self._emitted = i + 1
                row = torch.as_tensor(buf[i], dtype=torch.long)
                yield {"input_ids": row, "data_id": self.data_id} if self.return_data_id else row
            skip = 0
            if nxt is None:
                self._start, self._emitted, self._fill_rng = (len(self.parquet_files), 0), 0, after_rng
                return
            self._start, self._emitted, self._fill_rng = nxt, 0, after_rng

    def iter_batches(self, batch_size: int = 128):
        """Unshuffled token batches straight from the files (a sanity path that bypasses the buffer)."""
        import pyarrow.parquet as pq

        for f in self.parquet_files:
            for rb in pq.ParquetFile(f).iter_batches(batch_size=batch_size, columns=[self.column], use_threads=False):
                yield torch.as_tensor(rb.column(0).to_pylist(), dtype=torch.long)

    def state_dict(self):
        return {"start": tuple(self._start), "emitted": self._emitted, "fill_rng": self._fill_rng,
                "fingerprint": self.fingerprint}

    def load_state_dict(self, sd, **_):
        if sd.get("fingerprint") != self.fingerprint:
            print(f"WARNING dataset fingerprint mismatch: expected {self.fingerprint}, got {sd.get('fingerprint')}")
            return
        self._start, self._emitted = tuple(sd["start"]), int(sd["emitted"])
        st = sd["fill_rng"]
        self._fill_rng = (st[0], tuple(st[1]), st[2]) if not isinstance(st[1], tuple) else st

    load_local_state = load_state_dict


def _load_rows(path: str):
    """Rows of an on-disk text dataset: a parquet file or folder, a ``.jsonl`` file, or -- when the ``datasets`` package
    is installed -- an arrow folder written by ``save_to_disk``."""
    pth = Path(path)
    if pth.suffix == ".jsonl":
        import json

        with open(pth) as f:
            return [json.loads(line) for line in f if line.strip()]
    files = [pth] if pth.suffix == ".parquet" else sorted(pth.glob("*.parquet"))
    if files:
        import pyarrow.parquet as pq

        rows: list = []
        for f in files:
            rows.extend(pq.read_table(f).to_pylist())
        return rows
    import datasets

    ds = datasets.load_from_disk(str(pth))
    if isinstance(ds, datasets.DatasetDict):
        raise ValueError("the dataset path must point to a single split (try adding /train)")
    return ds


class TextRows(IterableDataset):
    """The ``hfds`` source: rows (dicts) of a map-style dataset, dealt out row by row -- not file by file -- over
    ``ranks x loader workers`` (shard ``rank * workers + worker`` takes rows ``shard::n_shards``), optionally repeated
    ``repetitions`` times; tokenisation happens in the collate function, driven by the ``data_signature`` attached to
    every row.  The position (``data_idx`` within this shard) is the resumable state
    (recpre/huggingface_dataset.py:297-441)."""

    def __init__(self, rows_or_path=None, data_signature: dict | None = None, num_processes: int = 1,
                 process_rank: int = 0, shuffle: bool = False, seed: int = 12345, data_id=None,
                 repetitions: int | None = None, return_data_id: bool | None = None, ds_name_or_path=None):
        rows_or_path = ds_name_or_path if rows_or_path is None else rows_or_path     # the reference's argument name
        assert rows_or_path is not None, "rows (a sequence of dicts) or the path of a saved dataset"
        if data_signature is None:
            data_signature = {"keys": ["text"], "format_fn": "pass_text"}
        if isinstance(rows_or_path, (str, Path)):
            rows_or_path = _load_rows(str(rows_or_path))
        self.rows, self.sig = rows_or_path, data_signature
        self.world, self.rank, self.shuffle, self.seed, self.data_id = num_processes, process_rank, shuffle, seed, data_id
        self.repetitions = max(1, int(repetitions or 1))
        self.return_data_id = (data_id is not None) if return_data_id is None else return_data_id
        self._pos = 0
        self.fingerprint, self.index_range = None, (0, 0)

    def _order(self) -> list:
        info = torch.utils.data.get_worker_info()
        workers, worker = (info.num_workers, info.id) if info is not None else (1, 0)
        total = len(self.rows) * self.repetitions
        order = list(range(self.rank * workers + worker, total, self.world * workers))
        if order:
            self.fingerprint = hashlib.shake_128(str(order).encode()).hexdigest(4)
            self.index_range = (order[0], order[-1])
        if self.shuffle:
            random.Random(self.seed).shuffle(order)
        return order

    def __len__(self) -> int:
        return len(self._order())

    def __iter__(self):
        order = self._order()
        n = len(self.rows)
        while self._pos < len(order):
            row = self.rows[order[self._pos] % n]
            self._pos += 1
            keys = self.sig.get("keys") if isinstance(self.sig, dict) else None
            row = {k: row[k] for k in keys} if keys and all(k in row for k in keys) else dict(row)
            row["data_signature"] = self.sig
            if self.return_data_id and self.data_id is not None:
                row["data_id"] = self.data_id
            yield row

    def state_dict(self):
        return {"pos": self._pos, "data_idx": self._pos}

    def load_state_dict(self, sd, **_):
        self._pos = int(sd.get("pos", sd.get("data_idx", 0)))

    load_local_state = load_state_dict


HuggingfaceDataset = TextRows      # the reference's class name for this source


class WeightedMixture(IterableDataset):
    """Draws the next row from one of several sources according to (scheduled) weights."""

    def __init__(self, sources: list | None = None, weights=None, seed=0, scheduler=None, *, datasets: list | None = None,
                 data_telemetry: bool = False):
        """``WeightedMixture(sources, weights, seed, scheduler)``; the reference's call
        ``HuggingfaceCombinedDataset(datasets, seed, weights=None, data_telemetry=False)`` is accepted as well
        (recpre/huggingface_dataset.py:444-481): an integer in second place is the seed, missing weights are uniform,
        telemetry prints the source of the first draws."""
        sources = datasets if sources is None else sources
        if isinstance(weights, int) and not isinstance(weights, bool):       # (datasets, seed, weights)
            weights, seed = (seed if isinstance(seed, (list, tuple)) else None), weights
        if weights is None:
            weights = [1.0 / len(sources)] * len(sources)
        self.sources, self.weights, self.scheduler = sources, list(weights), scheduler
        self.data_telemetry, self._draws = data_telemetry, 0
        self._rng = random.Random(seed)

    def __iter__(self):
        iters = [iter(s) for s in self.sources]
        alive = [True] * len(iters)
        while any(alive):
            w = self.scheduler.get_data_weights() if self.scheduler is not None else self.weights
            w = [wi if a else 0.0 for wi, a in zip(w, alive)]
            if sum(w) <= 0:
                return
            i = self._rng.choices(range(len(iters)), weights=w)[0]
            self._draws += 1
            if self.data_telemetry and self._draws <= 5:
                src = self.sources[i]
                print(f"draw {self._draws}: source {i} ({getattr(src, 'data_id', None)}:"
                      f"{getattr(src, 'fingerprint', None)})" if self._draws < 5 else "data telemetry off ...", flush=True)
            try:
                yield next(iters[i])
            except StopIteration:
                alive[i] = False

    def local_state(self):
        from .loader import local_state

        return {"sources": [local_state(s) for s in self.sources], "rng": self._rng.getstate()}

    def state_from_local(self, local):
        from .loader import saved_state

        return {"sources": [saved_state(s, l) for s, l in zip(self.sources, local["sources"])], "rng": local["rng"]}

    def state_dict(self):
        return self.state_from_local(self.local_state())

    def load_local_state(self, local) -> None:
        for s, st in zip(self.sources, local["sources"]):
            if st is not None and hasattr(s, "load_local_state"):
                s.load_local_state(st)
        self._rng.setstate(local["rng"])

    def load_state_dict(self, sd, **_):
        for s, st in zip(self.sources, sd["sources"]):
            if st is not None:
                s.load_state_dict(st)
        self._rng.setstate(sd["rng"])
