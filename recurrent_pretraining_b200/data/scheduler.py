"""Per-source sampling-weight schedules for data mixtures (recpre/data_scheduler_utils.py:1-229).

A source's ``scheduler`` entry is ``["const", w]``, ``["step", w0, every, gamma]``, ``["linear", w0, w1[, steps]]``,
``["cosine", w_max, w_min, period]``, ``["base"]`` / ``["base-renorm"]`` (this source takes what is left of 100), or
a piecewise list ``[[start_step, spec], ...]``.  A source whose ``max_epoch`` is exhausted gets weight 0.
"""
from __future__ import annotations

import math


def _make(spec, default_weight, max_steps):
    if isinstance(spec[0], (list, tuple)):
        pieces = [(int(start), _make(sub, default_weight, max_steps)) for start, sub in spec]

        def piecewise(step):
            for i, (start, fn) in enumerate(pieces):
                end = pieces[i + 1][0] if i + 1 < len(pieces) else float("inf")
                if start <= step < end:
                    return fn(step - start)
            return default_weight

        return piecewise
    kind = spec[0]
    if kind == "const":
        return lambda step: spec[1]
    if kind == "step":
        return lambda step: spec[1] * spec[3] ** (step // spec[2])
    if kind == "linear":
        total = spec[3] if len(spec) > 3 else max_steps
        return lambda step: spec[1] + (spec[2] - spec[1]) * (min(step, total) / total)
    if kind == "cosine":
        return lambda step: spec[2] + (spec[1] - spec[2]) * (1 + math.cos(math.pi * (step % spec[3]) / spec[3])) / 2
    if kind in ("base", "base-renorm"):
        return lambda step: 0
    raise NotImplementedError(f"unknown weight schedule {kind!r}")


class _Weight:
    """A weight schedule as an object with ``get_weight(step)``: the form in which the reference exposes its schedules
    (recpre/data_scheduler_utils.py:5-123).  The arithmetic is that of ``_make``; these classes only name it."""

    kind = ""

    def __init__(self, *args, max_steps: int = 0, default_weight=0):
        self.args = list(args)
        self._fn = _make([self.kind, *args], default_weight, max_steps)

    def get_weight(self, current_step: int):
        return self._fn(current_step)

    def __repr__(self):
        return f"{type(self).__name__}: {', '.join(str(a) for a in self.args)}"


class ConstWeight(_Weight):
    kind = "const"                                   # ConstWeight(weight)


class StepWeight(_Weight):
    kind = "step"                                    # StepWeight(initial_weight, step_size, gamma)


class LinearWeight(_Weight):
    kind = "linear"                                  # LinearWeight(initial_weight, end_weight, total_steps)


class CosineAnnealingWeight(_Weight):
    kind = "cosine"                                  # CosineAnnealingWeight(initial_weight, eta_min, T_max)


class BaseWeight(_Weight):
    kind = "base"                                    # the source that takes what the others leave of 100

    def get_weight(self, current_step: int):
        return 0


class PiecewiseWeight:
    """``[[start_step, spec], ...]``: each piece runs on its own clock from its start step."""

    def __init__(self, scheduler_configs, default_weight, max_steps: int = 0):
        self.scheduler_configs, self.default_weight = scheduler_configs, default_weight
        self._fn = _make(scheduler_configs, default_weight, max_steps)

    def get_weight(self, current_step: int):
        return self._fn(current_step)

    def __repr__(self):
        return f"PiecewiseWeight: {self.scheduler_configs}"


def GetScheduler(scheduler_config, default_weight, max_steps: int = 0):
    """Schedule object for one source's ``scheduler`` entry (None: constant at ``default_weight``)."""
    max_steps = int(getattr(max_steps, "max_steps", max_steps))      # the reference passes its settings object
    if scheduler_config is None:
        return ConstWeight(default_weight)
    if isinstance(scheduler_config[0], (list, tuple)):
        return PiecewiseWeight(scheduler_config, default_weight, max_steps)
    cls = {"const": ConstWeight, "step": StepWeight, "linear": LinearWeight, "cosine": CosineAnnealingWeight,
           "base": BaseWeight, "base-renorm": BaseWeight}.get(scheduler_config[0])
    if cls is None:
        raise NotImplementedError(f"unknown weight schedule {scheduler_config[0]!r}")
    return cls(*scheduler_config[1:], max_steps=max_steps, default_weight=default_weight)


class DataSchedulerTracker:
    def __init__(self, weights):
        self.weights = list(weights)
        self.sample_count = [0] * len(weights)
        self.epoch_count = [0] * len(weights)
        self.max_epochs = None
        self.base_id = None

    def reset(self):
        self.sample_count = [0] * len(self.weights)
        self.epoch_count = [0] * len(self.weights)

    def get_data_weights(self):
        return self.weights

    def get_sample_count(self):
        return self.sample_count

    def get_epoch_count(self):
        return self.epoch_count

    def __repr__(self):
        return (f"DataSchedulerTracker: {self.weights} | sample_count: {self.sample_count} | "
                f"epoch_count: {self.epoch_count}")


class DataScheduler:
    def __init__(self, tracker: DataSchedulerTracker = None, data_config: list = None, max_steps: int = 0, *,
                 data_scheduler_tracker: DataSchedulerTracker = None, args=None):
        """``DataScheduler(tracker, data_config, max_steps)``; the reference's keywords ``data_scheduler_tracker`` and
        ``args`` (an object with ``max_steps``) are accepted too (recpre/data_scheduler_utils.py:150-170)."""
        tracker = data_scheduler_tracker if tracker is None else tracker
        if not isinstance(max_steps, int):               # (tracker, data_config, args) passed positionally
            args, max_steps = max_steps, 0
        if args is not None:
            max_steps = int(getattr(args, "max_steps", max_steps))
        self.tracker = tracker
        self.base_id, self._renorm = None, False
        self.max_epochs, self._fns = [], []
        for i, entry in enumerate(data_config):
            self.max_epochs.append(entry.max_epoch if entry.max_epoch is not None else float("inf"))
            spec = entry.scheduler if entry.scheduler is not None else ["const", entry.weight]
            if spec[0] in ("base", "base-renorm"):
                self.base_id = i
                tracker.base_id = i
                self._renorm = spec[0] == "base-renorm"
            self._fns.append(_make(spec, entry.weight, max_steps))
        tracker.max_epochs = self.max_epochs

    def step(self, curr_step: int) -> None:
        w = [fn(curr_step) for fn in self._fns]
        for i in range(len(w)):
            if self.max_epochs[i] <= self.tracker.epoch_count[i]:
                w[i] = 0
        if self.base_id is not None:
            explicit = sum(x for i, x in enumerate(w) if i != self.base_id)
            if self._renorm and explicit != 0:
                w = [x * 100.0 / explicit if i != self.base_id else 0 for i, x in enumerate(w)]
            w[self.base_id] = 0
            w[self.base_id] = 100.0 - sum(w)
        self.tracker.weights[:] = w

    def get_data_weights(self):
        return self.tracker.weights

    def get_sample_count(self):
        return self.tracker.sample_count

    def get_epoch_count(self):
        return self.tracker.epoch_count

    def __repr__(self):
        return f"DataScheduler(weights={self.tracker.weights}, max_epochs={self.max_epochs}, base={self.base_id})"

    def set_one_hot_schedule(self, idx: int) -> None:
        self._fns = [(lambda s: 0) for _ in self._fns]
        self._fns[idx] = lambda s: 1

    def state_dict(self):
        return {"weights": list(self.tracker.weights), "sample_count": list(self.tracker.sample_count),
                "epoch_count": list(self.tracker.epoch_count)}

    def load_state_dict(self, sd):
        self.tracker.weights[:] = sd["weights"]
        self.tracker.sample_count = list(sd["sample_count"])
        self.tracker.epoch_count = list(sd["epoch_count"])
