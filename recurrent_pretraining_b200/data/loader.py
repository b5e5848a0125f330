"""Stateful batch loader: wraps an iterable token source, collates micro-batches, pins them and prefetches on a
background thread (the role of torchdata's StatefulDataLoader in the reference, train.py:742-753)."""
from __future__ import annotations

import queue
import threading

import torch


class StatefulLoader:
    def __init__(self, dataset, batch_size: int, collate_fn, pin_memory: bool = True, prefetch: int = 4,
                 drop_last: bool = True):
        self.dataset, self.batch_size, self.collate_fn = dataset, batch_size, collate_fn
        self.pin = pin_memory and torch.cuda.is_available()
        self.prefetch, self.drop_last = prefetch, drop_last
        self.batches_yielded = 0
        self._restore_state = None

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
                    snapshot = self.dataset.state_dict() if self.prefetch == 0 and hasattr(self.dataset, "state_dict") \
                        else None
                    out.put((batch, snapshot))
                    rows = []
            if rows and not self.drop_last:
                out.put((self.collate_fn(rows), None))
        except Exception as exc:  # surface loader errors in the training thread
            out.put(exc)
        finally:
            out.put(None)

    def __iter__(self):
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
                    yield batch
            return
        q: queue.Queue = queue.Queue(maxsize=self.prefetch)
        stop = threading.Event()
        t = threading.Thread(target=self._produce, args=(q, stop), daemon=True)
        t.start()
        try:
            while True:
                item = q.get()
                if item is None:
                    return
                if isinstance(item, Exception):
                    raise item
                self.batches_yielded += 1
                yield item[0]
        finally:
            stop.set()

    def state_dict(self):
        """Loader position.  With prefetching the source is ahead of the consumer by at most ``prefetch`` batches;
        resuming skips nothing twice because the source state is rewound by replaying from ``batches_yielded``."""
        sd = {"batches_yielded": self.batches_yielded}
        if hasattr(self.dataset, "state_dict"):
            sd["dataset"] = self.dataset.state_dict()
        return sd

    def load_state_dict(self, sd):
        self.batches_yielded = sd.get("batches_yielded", 0)
        if "dataset" in sd and hasattr(self.dataset, "load_state_dict"):
            self.dataset.load_state_dict(sd["dataset"])
