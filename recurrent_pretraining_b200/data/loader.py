"""Stateful batch loader: wraps an iterable token source, collates micro-batches, pins them and prefetches on a
background thread (the role of torchdata's StatefulDataLoader in the reference, train.py:742-753).

Resume is exact with prefetching: the producer thread takes a (non-collective) snapshot of the source right after the
last row of every batch has been drawn and queues it with the batch; ``state_dict`` returns the snapshot that belongs
to the last batch the consumer received, so batches that were prefetched but never trained on are produced again after a
resume.  Collectives that a source needs to assemble its saved state (the per-rank gather of the parquet stream) run in
``state_dict``, on the calling thread, never on the producer thread.
"""
from __future__ import annotations

import queue
import threading

import torch


def local_state(ds):
    """Snapshot of a source without any collective."""
    if hasattr(ds, "local_state"):
        return ds.local_state()
    if hasattr(ds, "state_dict"):
        return ds.state_dict()
    return None


def saved_state(ds, local):
    """The form of ``local`` that goes into a checkpoint (a source may gather it over ranks here)."""
    if local is None:
        return None
    if hasattr(ds, "state_from_local"):
        return ds.state_from_local(local)
    return local


class StatefulLoader:
    def __init__(self, dataset, batch_size: int, collate_fn, pin_memory: bool = True, prefetch: int = 4,
                 drop_last: bool = True):
        self.dataset, self.batch_size, self.collate_fn = dataset, batch_size, collate_fn
        self.pin = pin_memory and torch.cuda.is_available()
        self.prefetch, self.drop_last = prefetch, drop_last
        self.batches_yielded = 0
        self._snapshot = None        # source state after the last batch handed to the consumer
        self._running = False

    def _produce(self, out: queue.Queue, stop: threading.Event):
        try:
            rows = []
            for row in self.dataset:
                if stop.is_set():
                    return
                rows.append(row)
                if len(rows) == self.batch_size:
                    try:
                        batch = self.collate_fn(rows)
                    except StopIteration:
                        break
                    if self.pin:
                        batch = tuple(t.pin_memory() if torch.is_tensor(t) else t for t in batch)
                    # the source generator is suspended at its yield: this snapshot is exactly "after this batch"
                    snapshot = local_state(self.dataset)
                    while not stop.is_set():
                        try:
                            out.put((batch, snapshot), timeout=0.2)
                            break
                        except queue.Full:
                            continue
                    rows = []
            if rows and not self.drop_last and not stop.is_set():
                out.put((self.collate_fn(rows), local_state(self.dataset)))
        except Exception as exc:  # surface loader errors in the training thread
            out.put(exc)
        finally:
            try:
                out.put(None, timeout=1.0)
            except queue.Full:
                pass

    def __iter__(self):
        if self._snapshot is None:
            self._snapshot = local_state(self.dataset)
        if self.prefetch <= 0:
            rows = []
            for row in self.dataset:
                rows.append(row)
                if len(rows) == self.batch_size:
                    try:
                        batch = self.collate_fn(rows)
                    except StopIteration:
                        return
                    rows = []
                    self.batches_yielded += 1
                    self._snapshot = local_state(self.dataset)
                    yield batch
            return
        q: queue.Queue = queue.Queue(maxsize=self.prefetch)
        stop = threading.Event()
        t = threading.Thread(target=self._produce, args=(q, stop), daemon=True)
        self._running = True
        t.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    return
                if isinstance(item, Exception):
                    raise item
                self.batches_yielded += 1
                self._snapshot = item[1]
                yield item[0]
        finally:
            stop.set()
            self._running = False
            t.join(timeout=5.0)
            # the producer ran ahead of the consumer: put the source back to where the consumer stopped
            if self._snapshot is not None and hasattr(self.dataset, "load_local_state"):
                self.dataset.load_local_state(self._snapshot)

    def state_dict(self):
        """Loader position: the source state that belongs to the last batch the consumer received."""
        snap = self._snapshot if (self._snapshot is not None or self._running) else local_state(self.dataset)
        sd = {"batches_yielded": self.batches_yielded}
        saved = saved_state(self.dataset, snap)
        if saved is not None:
            sd["dataset"] = saved
        return sd

    def load_state_dict(self, sd):
        self.batches_yielded = sd.get("batches_yielded", 0)
        if "dataset" in sd and hasattr(self.dataset, "load_state_dict"):
            self.dataset.load_state_dict(sd["dataset"])
        self._snapshot = local_state(self.dataset)
