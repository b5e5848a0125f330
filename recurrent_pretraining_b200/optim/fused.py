"""Fused flat-buffer Adam family for the GPU path.

One kernel launch per optimizer group (or per bucket of tensors in the sharded step) does: global-norm clip (factor
derived on the device from the reduced squared norm), weight decay, both moment updates, the parameter update in
fp32, and the bf16 compute copy.  No host synchronisation: a non-finite norm turns the launch into a no-op on the
device (train.py:446-461 of the reference skips such steps on the host).

Semantics: ``torch.optim.AdamW`` (recpre/optim.py:115-120) by default.  The flags select the options of the
reference's ELLISAdam that its production run enables (recpre/optim.py:803-840,949-1019;
launch_configs/frontier_nebel_512_nodes.yaml:28-41):

* ``atan2``            ``p -= step * atan2(m, sqrt(v) / sqrt(1 - b2^t))`` instead of the division by ``sqrt(v) + eps``
* ``update_clipping``  per tensor: ``v`` is clamped to ``eps^2`` and ``step = lr / max(1, sqrt(mean(g^2 / v)))``
* ``running_init``     both moments start at the first gradient (``m = g, v = g^2``) instead of zero
* ``decouple_wd``      decay factor ``1 - lr / lr0 * wd`` relative to the constructor learning rate ``lr0``

Optimizer state can be sharded: ``attach_plans`` gives every group a ``GroupShards`` description and this rank keeps
``m`` and ``v`` only for its own piece of every tensor, concatenated in tensor order.
"""
from __future__ import annotations

import math
import os

import torch

from ..ops import reference as ref


def deferred_runs(names, offsets, numels, total: int):
    """Cut a flat weight group into contiguous runs ``(phase, lo, hi)`` in buffer order, ``phase`` being ``"core"`` /
    ``"coda"`` for the tensors the forward pass needs late and ``None`` for the rest.  Returns None unless the core and
    the coda are ONE run each.  Alignment gaps are covered: every run ends where the next begins."""
    from ..parallel.segments import bucket_of

    runs: list = []
    for name, off, n in sorted(zip(names, offsets, numels), key=lambda x: x[1]):
        head = bucket_of(name, "weight").split(".")[0]
        phase = head if head in ("core", "coda") else None
        if runs and runs[-1][0] == phase:
            runs[-1][2] = off + n
        else:
            runs.append([phase, off, off + n])
    if sorted(r[0] for r in runs if r[0]) != ["coda", "core"]:
        return None
    for a, b in zip(runs, runs[1:]):
        a[2] = b[1]
    runs[0][1], runs[-1][2] = 0, total
    return [tuple(r) for r in runs]


class FusedAdamW:
    def __init__(self, flat_groups, lr=4e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, atan2=False,
                 update_clipping=False, running_init=False, decouple_wd=False):
        self.groups = flat_groups
        self.defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        self.atan2, self.update_clipping = bool(atan2), bool(update_clipping)
        self.running_init, self.decouple_wd = bool(running_init), bool(decouple_wd)
        self.step_count = 0
        self.param_groups = []
        self.rank, self.world = 0, 1
        self.plans = None
        for g in flat_groups:
            h = dict(self.defaults)
            h.update(g.hyper)
            h["params"] = g.params
            h["init_lr"] = float(lr)     # the constructor value, as in the reference (recpre/optim.py:744)
            self.param_groups.append(h)
            g.state["m"] = torch.zeros_like(g.master)
            g.state["v"] = torch.zeros_like(g.master)
            g.state["range"] = (0, g.numel)
        dev = flat_groups[0].master.device
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=dev)

    @property
    def plain_adamw(self) -> bool:
        return not (self.update_clipping or self.running_init or self.decouple_wd)

    def decay_factor(self, h) -> float:
        lr = float(h["lr"])
        if self.decouple_wd:
            return 1.0 - lr / max(h["init_lr"], 1e-30) * h["weight_decay"]
        return 1.0 - lr * h["weight_decay"]

    # -- sharding --------------------------------------------------------------------------
    def shard(self, ranges) -> None:
        """Keep optimizer state only for ``ranges[i] = (lo, hi)`` of group i (contiguous-range sharding)."""
        for g, (lo, hi) in zip(self.groups, ranges):
            dev = g.master.device
            g.state["m"] = torch.zeros(max(hi - lo, 4), dtype=torch.float32, device=dev)
            g.state["v"] = torch.zeros(max(hi - lo, 4), dtype=torch.float32, device=dev)
            g.state["range"] = (lo, hi)

    defer_ranges = None

    def attach_plans(self, plans, rank: int, world: int) -> None:
        """Per-tensor sharding: this rank keeps the moments of its own piece of every tensor (``plans[i]`` is the
        ``GroupShards`` of group i), concatenated in tensor order."""
        self.plans, self.rank, self.world = plans, rank, world
        for g, plan in zip(self.groups, plans):
            dev = g.master.device
            n = max(plan.owned(rank), 4)
            g.state["m"] = torch.zeros(n, dtype=torch.float32, device=dev)
            g.state["v"] = torch.zeros(n, dtype=torch.float32, device=dev)
            g.state["range"] = None

    # -- norm ------------------------------------------------------------------------------
    def compute_grad_norm_sq(self) -> torch.Tensor:
        self.gnorm_sq.zero_()
        if self.gnorm_sq.is_cuda:
            from ..ops import cuda as C

            for g in self.groups:
                C.sumsq_(g.grad, self.gnorm_sq)
        else:
            for g in self.groups:
                self.gnorm_sq += g.grad.pow(2).sum()
        return self.gnorm_sq

    # -- reference update of one piece (CPU path and oracle of the kernels) -----------------
    def update_piece(self, p, g, m, v, h, step: int, gscale: float, first_update: bool, rms_sq_mean=None):
        """In-place update of fp32 tensors of equal shape.  ``rms_sq_mean`` is mean(g^2 / v) over the WHOLE tensor
        (update clipping), or None."""
        b1, b2 = h["betas"]
        lr, eps = float(h["lr"]), h["eps"]
        g = g * gscale
        if self.running_init and first_update:
            m.copy_(g)
            v.copy_(g * g)
        m.lerp_(g, 1 - b1)
        v.mul_(b2).addcmul_(g, g, value=1 - b2)
        step_size = lr
        if self.update_clipping:
            v.clamp_(min=eps ** 2)
            step_size = lr / max(math.sqrt(float(rms_sq_mean)), 1.0)
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        step_size = step_size / bc1
        p.mul_(self.decay_factor(h))
        if self.atan2:
            p.add_(torch.atan2(m, v.sqrt() / math.sqrt(bc2)), alpha=-step_size)
        else:
            p.addcdiv_(m, (v.sqrt() / math.sqrt(bc2)).add_(eps), value=-step_size)

    def clip_stat(self, g, v, h, gscale: float, first_update: bool) -> torch.Tensor:
        """sum(g^2 / max(v', eps^2)) of one piece, v' being the second moment after this step's update."""
        b2 = h["betas"][1]
        g2 = (g * gscale).pow(2)
        vn = g2 if (self.running_init and first_update) else v * b2 + g2 * (1 - b2)
        return (g2 / vn.clamp(min=h["eps"] ** 2)).sum()

    # -- step ------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, max_norm: float = 0.0, grad_scale: float = 1.0, zero_grad: bool = True, norm_ready: bool = False):
        """Replicated update of all groups on full-size state (one process, or after an all-reduce).  ``gnorm_sq`` must
        hold the squared norm of the *stored* gradients (before ``grad_scale``) unless clipping is off; it is computed
        here when ``norm_ready`` is False."""
        assert self.plans is None, "sharded state is stepped by parallel.p2p.ShardedStepper"
        self.finish_deferred()       # a step that follows another without a forward pass in between
        if not norm_ready:
            self.compute_grad_norm_sq()
        first_update = self.step_count == 0
        self.step_count += 1
        on_gpu = self.groups[0].master.is_cuda
        if on_gpu and not self.plain_adamw:
            from ..parallel.p2p import single_device_table_step

            single_device_table_step(self, max_norm, grad_scale, zero_grad, first_update)
            return
        clip = 1.0
        if not on_gpu:
            gn = float(self.gnorm_sq.sqrt()) * grad_scale
            if not math.isfinite(gn):
                if zero_grad:
                    self.zero_grad()
                return
            clip = min(1.0, max_norm / (gn + 1e-6)) if max_norm > 0 else 1.0
        later = []
        for gi, (g, h) in enumerate(zip(self.groups, self.param_groups)):
            lr = float(h["lr"])
            b1, b2 = h["betas"]
            if on_gpu:
                from ..ops import cuda as C

                def run(lo, hi, g=g, h=h, lr=lr, b1=b1, b2=b2):
                    sl = slice(lo, hi)
                    C.adamw_(g.master[sl], g.grad[sl], g.state["m"][sl], g.state["v"][sl],
                             g.shadow[sl] if g.shadow is not None else None, self.gnorm_sq, lr=lr, beta1=b1,
                             beta2=b2, eps=h["eps"], wd=h["weight_decay"], step=self.step_count, max_norm=max_norm,
                             grad_scale=grad_scale, zero_grad=zero_grad, atan2=self.atan2)

                ranges = self.defer_ranges.get(gi) if self.defer_ranges else None
                if not ranges:
                    run(0, g.master.numel())
                    continue
                for phase, lo, hi in ranges:
                    if phase is None:
                        run(lo, hi)
                    else:
                        later.append((phase, lo, hi, run))
                continue
            if self.plain_adamw and not self.atan2:
                ref.adamw_step(g.master, g.grad, g.state["m"], g.state["v"], lr, b1, b2, h["eps"], h["weight_decay"],
                               self.step_count, grad_scale * clip)
            else:
                for p, off in zip(g.params, g.offsets):
                    n = p.numel()
                    sl = slice(off, off + n)
                    stat = None
                    if self.update_clipping:
                        stat = self.clip_stat(g.grad[sl], g.state["v"][sl], h, grad_scale * clip, first_update) / n
                    self.update_piece(g.master[sl], g.grad[sl], g.state["m"][sl], g.state["v"][sl], h,
                                      self.step_count, grad_scale * clip, first_update, stat)
            if g.shadow is not None:
                g.shadow.copy_(g.master)
            if zero_grad:
                g.grad.zero_()
        if later:
            self._run_deferred(later)

    # -- deferred part of the single-GPU update ------------------------------------------------
    def enable_deferred(self, model) -> bool:
        """One GPU, plain AdamW: update the weights the next forward pass needs late (recurrent core, coda) on a side
        stream beside that pass's first layers; the update is bound by HBM, those layers by the tensor cores.  The model
        waits at its ``core`` / ``coda`` points (``on_forward``); other readers call ``finish_deferred``.  Needs the
        core and the coda tensors to be contiguous runs of the flat weight group (module order gives that)."""
        self.defer_ranges = None
        if self.plans is not None or not self.plain_adamw or not self.groups[0].master.is_cuda \
                or not hasattr(model, "_fwd_point") or os.environ.get("B200_DEFER_UPDATE", "1") != "1":
            return False
        g = self.groups[0]
        runs = deferred_runs(g.names, g.offsets, [p.numel() for p in g.params], g.master.numel())
        if runs is None:
            return False
        self.defer_ranges = {0: runs}
        self._side = torch.cuda.Stream(device=g.master.device, priority=-1)
        self._deferred_events = {}
        model._fwd_cb = self.on_forward
        return True

    def _run_deferred(self, later) -> None:
        self.finish_deferred()
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self._side.wait_event(ev)
        order = {"core": 0, "coda": 1}
        with torch.cuda.stream(self._side):
            for phase, lo, hi, run in sorted(later, key=lambda x: order[x[0]]):
                run(lo, hi)
                done = torch.cuda.Event()
                done.record(self._side)
                self._deferred_events[phase] = done

    def on_forward(self, name: str) -> None:
        ev = self._deferred_events.pop(name, None) if self.defer_ranges else None
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def finish_deferred(self) -> None:
        if self.defer_ranges:
            for name in list(self._deferred_events):
                self.on_forward(name)

    def grad_norm(self, grad_scale: float = 1.0) -> torch.Tensor:
        return self.gnorm_sq.sqrt() * grad_scale

    def zero_grad(self, set_to_none: bool = False):
        self.finish_deferred()       # the deferred part of the last update still reads its gradients
        for g in self.groups:
            g.grad.zero_()

    # -- checkpoint --------------------------------------------------------------------------
    def state_dict(self):
        self.finish_deferred()
        groups = []
        for gi, (g, h) in enumerate(zip(self.groups, self.param_groups)):
            entry = {"m": g.state["m"], "v": g.state["v"], "range": g.state["range"], "names": g.names,
                     "offsets": g.offsets, "numel": g.numel,
                     "hyper": {k: v for k, v in h.items() if k != "params"}}
            if self.plans is not None:
                plan = self.plans[gi]
                entry["shards"] = {"numels": plan.numels, "pers": plan.pers, "rank": self.rank, "world": self.world}
            groups.append(entry)
        return {"step": self.step_count, "groups": groups}

    def _layout(self, gi: int):
        if self.plans is None:
            return None
        plan = self.plans[gi]
        return {"numels": list(plan.numels), "pers": list(plan.pers), "rank": self.rank, "world": self.world}

    def load_state_dict(self, sd, other_shards=None):
        """``other_shards``: callable returning the optimizer state dicts of ALL ranks of the saved run (used to
        rebuild this rank's pieces when the saved sharding differs from the current one)."""
        self.step_count = sd["step"]
        for gi, (g, h, s) in enumerate(zip(self.groups, self.param_groups, sd["groups"])):
            saved, now = s.get("shards"), self._layout(gi)
            if list(s.get("names", g.names)) != list(g.names):
                raise ValueError(f"optimizer group {gi}: parameter names differ from the checkpoint")
            same = (saved is None and now is None and tuple(s["m"].shape) == tuple(g.state["m"].shape)) or \
                   (saved is not None and now is not None and saved == now)
            if same:
                g.state["m"].copy_(s["m"])
                g.state["v"].copy_(s["v"])
            else:
                m_full, v_full = self._assemble_full(gi, sd, other_shards)
                self._take_from_full(gi, m_full, v_full)
            for k, v in s.get("hyper", {}).items():
                h[k] = v

    def _assemble_full(self, gi: int, sd, other_shards):
        """Full-size (flat-buffer layout) moments of group ``gi`` from the saved run's shards."""
        s = sd["groups"][gi]
        numel = s.get("numel", self.groups[gi].numel)
        if s.get("shards") is None:
            if s.get("range") not in (None, (0, numel)) and tuple(s.get("range")) != (0, numel):
                raise ValueError("checkpoint holds a contiguous-range optimizer shard; resume with the world size it "
                                 "was written with")
            return s["m"].float().cpu(), s["v"].float().cpu()
        if other_shards is None:
            raise ValueError(f"optimizer group {gi} was saved with sharding {s['shards']['world']} ways; the other "
                             "ranks' files are needed to re-shard it")
        all_sd = other_shards()
        world = s["shards"]["world"]
        if len(all_sd) != world:
            raise ValueError(f"found {len(all_sd)} of {world} optimizer shards")
        m_full = torch.zeros(numel, dtype=torch.float32)
        v_full = torch.zeros(numel, dtype=torch.float32)
        for osd in all_sd:
            e = osd["groups"][gi]
            q, pers, numels = e["shards"]["rank"], e["shards"]["pers"], e["shards"]["numels"]
            acc = 0
            for t, off in enumerate(e["offsets"]):
                lo = min(q * pers[t], numels[t])
                hi = min(lo + pers[t], numels[t])
                n = hi - lo
                m_full[off + lo:off + hi] = e["m"][acc:acc + n].float().cpu()
                v_full[off + lo:off + hi] = e["v"][acc:acc + n].float().cpu()
                acc += n
        return m_full, v_full

    def _take_from_full(self, gi: int, m_full, v_full) -> None:
        g = self.groups[gi]
        if self.plans is None:
            g.state["m"].copy_(m_full[:g.state["m"].numel()])
            g.state["v"].copy_(v_full[:g.state["v"].numel()])
            return
        plan = self.plans[gi]
        acc = 0
        for t in range(len(plan.offs)):
            start, n = plan.segment(t, self.rank)
            g.state["m"][acc:acc + n].copy_(m_full[start:start + n])
            g.state["v"][acc:acc + n].copy_(v_full[start:start + n])
            acc += n
