"""Sharded data-parallel optimizer step with hand-written NVLink kernels, overlapped with the backward pass.

Gradients live in flat fp32 buffers in symmetric (peer-mapped) memory.  Every tensor is cut over all ranks
(``parallel/segments.py``); the tensors are grouped into buckets by the point of the backward pass at which their
gradients are complete: coda, recurrent core + adapter, prelude, and the rest (tied embedding / head, norm scales).
The model marks these points with tensor hooks; when one fires, the bucket's reduce-scatter is launched on a side
stream (a small number of CTAs, sharing the SMs with the GEMMs of the layers still going backward):

    [per bucket]  reduce-scatter kernel: its first CTA tells every peer "my gradients of this bucket are complete", all
                  CTAs wait (bounded) for the peers' signals, then sum the owner's pieces from all ranks and add to the
                  squared-norm partial
    [after backward]  barrier + exchange of the norm partials  ->  (ELLISAdam: per-tensor clipping statistics, barrier)
                  ->  update of the owned pieces (AdamW or the ELLISAdam flags) that writes the new bf16 compute copy
                  ->  barrier

Two modes.  ``dp``: every rank keeps full fp32 masters and bf16 compute copies; the update kernel stores the new bf16
values into every rank's copy (two-shot all-reduce whose second shot carries parameters).  ``zero3``: fp32 masters and
optimizer state exist only for the owned pieces; the update writes the owner's copy only, and the next forward pass
pulls the other ranks' pieces bucket by bucket on a side stream, the row-sharded QKV and gate-up weights inside the
first GEMM that consumes them (``b200_ag_gemm``).

This replaces the reference's post-backward chunked fp32 all-reduce, replicated clip and replicated (or ZeRO-1
broadcast) optimizer step (recpre/utils.py:1004-1043,1196-1206; recpre/optim.py:131-263).  A ``torch`` backend runs the
same bookkeeping with ``torch.distributed`` collectives (CPU / gloo) and is the oracle for the host-side logic.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import torch
import torch.distributed as dist

from ..utils import nvtx
from .segments import MAX_BUCKETS, GroupShards, bucket_of, gather_key, readiness_key
from .symm import SymmetricBuffer

ALIGN = 128
GROUP_KINDS = ("weight", "embedding", "norm")
SLOT_BYTES = 64            # one flag slot: 16 x uint32
CTRL_BYTES = 4096          # 32 flag slots, then two norm partials at byte 2048
PARTIAL_OFF = 2048


class OptArgsC(C.Structure):
    _fields_ = [(n, C.c_float) for n in ("lr", "beta1", "beta2", "eps", "decay", "bc1", "bc2", "max_norm",
                                         "grad_scale")] + \
               [(n, C.c_int) for n in ("atan2_mode", "update_clip", "state_init", "zero_grad", "n_push", "push_master",
                                       "master_sharded", "n_ranks", "max_ctas")]


def shard_range(numel: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous-range split of a flat buffer (communication sweep and older callers)."""
    per = (numel + world - 1) // world
    per = (per + ALIGN - 1) // ALIGN * ALIGN
    lo = min(rank * per, numel)
    return lo, min(lo + per, numel)


class P2PAllocator:
    """Hands out flat buffers that live in symmetric memory; remembers them per (group index, kind)."""

    def __init__(self, fabric):
        self.fabric = fabric
        self.buffers: dict = {}

    def __call__(self, group_index: int, kind: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        size = 4 if dtype == torch.float32 else 2
        buf = SymmetricBuffer(self.fabric, numel * size)
        self.buffers[(group_index, kind)] = buf
        return buf.tensor(dtype, numel)


def _opt_args(opt, h, *, max_norm, grad_scale, first_update, n_push, push_master, master_sharded, n_ranks,
              zero_grad=False, max_ctas=0) -> OptArgsC:
    b1, b2 = h["betas"]
    t = max(opt.step_count, 1)
    a = OptArgsC()
    a.lr, a.beta1, a.beta2, a.eps = float(h["lr"]), b1, b2, h["eps"]
    a.decay = opt.decay_factor(h)
    a.bc1, a.bc2 = 1.0 - b1 ** t, 1.0 - b2 ** t
    a.max_norm, a.grad_scale = max_norm, grad_scale
    a.atan2_mode, a.update_clip = int(opt.atan2), int(opt.update_clipping)
    a.state_init = int(opt.running_init and first_update)
    a.zero_grad, a.n_push, a.push_master = int(zero_grad), n_push, int(push_master)
    a.master_sharded, a.n_ranks = int(master_sharded), n_ranks
    a.max_ctas = int(max_ctas)
    return a


def single_device_table_step(opt, max_norm: float, grad_scale: float, zero_grad: bool, first_update: bool) -> None:
    """One-GPU update through the table kernels (the ELLISAdam flags); ``opt.gnorm_sq`` already holds the norm."""
    from ..ops import cuda as K

    dev = opt.groups[0].master.device
    st = C.c_void_p(K._stream())
    n_stats = sum(len(g.params) for g in opt.groups)
    stats = getattr(opt, "_stats", None)
    if stats is None or stats.numel() < n_stats:
        stats = opt._stats = torch.zeros(max(n_stats, 4), dtype=torch.float32, device=dev)
    plans = [GroupShards.plan(g, 1) for g in opt.groups]
    stat_ptr = (C.c_void_p * 1)(stats.data_ptr())
    base = 0
    launches = []
    for g, h, plan in zip(opt.groups, opt.param_groups, plans):
        a = _opt_args(opt, h, max_norm=max_norm, grad_scale=grad_scale, first_update=first_update, n_push=1,
                      push_master=False, master_sharded=False, n_ranks=1, zero_grad=zero_grad)
        for tb in plan.tables(range(len(g.params)), 0, base):
            launches.append((g, a, tb))
        base += len(g.params)
    if opt.update_clipping:
        stats.zero_()
        for g, a, tb in launches:
            K._check(K.lib.b200_opt_stats(C.c_void_p(g.grad.data_ptr()), C.c_void_p(g.state["v"].data_ptr()),
                                          C.byref(tb), 0, C.c_void_p(opt.gnorm_sq.data_ptr()), C.byref(a),
                                          C.c_void_p(stats.data_ptr()), st), "opt_stats")
    for g, a, tb in launches:
        shadow = (C.c_void_p * 1)(g.shadow.data_ptr() if g.shadow is not None else 0)
        K._check(K.lib.b200_opt_table(C.c_void_p(g.master.data_ptr()), C.c_void_p(g.grad.data_ptr()),
                                      C.c_void_p(g.state["m"].data_ptr()), C.c_void_p(g.state["v"].data_ptr()),
                                      shadow, None, stat_ptr, C.byref(tb), 0, C.c_void_p(opt.gnorm_sq.data_ptr()),
                                      C.byref(a), st), "opt_table")


class _Bucket:
    def __init__(self, name: str, slot: int):
        self.name, self.slot = name, slot
        self.tensors: dict = {}      # group index -> tensor indices
        self.tables: list = []       # (group index, table)
        self.params: list = []
        self.fired = False
        self.gather_event = None


class ShardedStepper:
    def __init__(self, fabric, groups, optimizer, model=None, *, zero3: bool = False, allocator: P2PAllocator | None = None,
                 backend: str | None = None, timeout_ms: int = 20000):
        self.fabric, self.groups, self.opt, self.alloc = fabric, groups, optimizer, allocator
        self.rank, self.world = fabric.global_rank, fabric.world_size
        self.zero3 = zero3
        self.backend = backend or ("cuda" if fabric.device.type == "cuda" else "torch")
        self.timeout_ms = timeout_ms
        self.epoch = 0
        self.reduce_count = 0
        self.overlap = os.environ.get("B200_OVERLAP", "1") == "1"
        self.overlap_ctas = int(os.environ.get("B200_RS_CTAS", "32"))
        # B200_TRACE=1: CUDA-event stamps of every bucket's reduce-scatter (side stream) against the step's main-stream
        # milestones, kept for the last step in ``self.trace`` (see ``timeline()``)
        self.tracing = os.environ.get("B200_TRACE", "0") == "1"
        self.trace: dict = {}
        self.plans = [getattr(g, "plan", None) or GroupShards.plan(g, self.world) for g in groups]
        optimizer.attach_plans(self.plans, self.rank, self.world)
        n_layer = getattr(getattr(model, "config", None), "n_layer", 0) if model is not None and \
            type(model).__name__ == "GPT" else 0
        # buckets -------------------------------------------------------------------------------
        def assign(coarse: bool) -> dict:
            found: dict = {}
            for gi, g in enumerate(groups):
                kind = GROUP_KINDS[gi] if gi < len(GROUP_KINDS) else "weight"
                for t, (name, p) in enumerate(zip(g.names, g.params)):
                    found.setdefault(bucket_of(name, kind, n_layer, coarse), []).append((gi, t, p))
            return found

        found = assign(False)
        if len(found) > MAX_BUCKETS:          # very deep prelude / coda: one bucket for each of them
            found = assign(True)
        self.order = sorted(found, key=readiness_key)            # completion order of the gradients
        self.gather_order = sorted(found, key=gather_key)        # order in which the forward pass needs the weights
        self.buckets: dict = {}
        for slot, bname in enumerate(self.order, start=1):
            b = self.buckets[bname] = _Bucket(bname, slot)
            for gi, t, p in found[bname]:
                b.tensors.setdefault(gi, []).append(t)
                b.params.append(p)
                p._bucket = b
        # a bucket fired by a hook shares the SMs with the backward pass of the layers before it and gets few CTAs; the
        # buckets whose hook comes when (almost) nothing is left to run get the whole machine
        self.full_width = set(self.order[-2:]) if len(self.order) > 1 else set(self.order)
        self.stat_base, base = [], 0
        for g in groups:
            self.stat_base.append(base)
            base += len(g.params)
        self.n_stats = base
        for b in self.buckets.values():
            for gi, ids in b.tensors.items():
                for tb in self.plans[gi].tables(ids, self.rank, self.stat_base[gi]):
                    b.tables.append((gi, tb))
        self.master_sharded = [bool(getattr(g, "master_sharded", False)) for g in groups]
        self.dirty = False         # zero3: owners hold newer pieces than the local copies
        # Deferred update (replicated-parameter mode): the weights of the recurrent core and of the coda are needed by
        # the next forward pass only after the prelude, so their update + push runs on the side stream beside the next
        # step's first layers instead of in the exposed tail of this step.  The forward pass waits at the model's
        # "core" / "coda" points (``on_forward``); every other reader of parameters calls ``finish_deferred``.
        self.defer = (os.environ.get("B200_DEFER_UPDATE", "1") == "1" and self.world > 1 and not zero3
                      and self.backend == "cuda" and "core" in self.buckets
                      and any(n.startswith("coda") for n in self.buckets))
        # the core's update must be over when the prelude's forward pass is (a few ms): full width, its CTAs share the
        # SMs with the prelude GEMMs; the coda's has the whole recurrence to hide in: few CTAs
        self.defer_ctas = {"core": int(os.environ.get("B200_DEFER_CTAS_CORE", "0")),
                           "coda": int(os.environ.get("B200_DEFER_CTAS_CODA", "32"))}
        self.deferred_events: dict = {}
        self.defer_epoch = 0
        if self.backend == "cuda":
            self._setup_cuda()
        if self.world > 1 and dist.is_initialized():
            if fabric.device.type == "cuda":
                dist.barrier(device_ids=[fabric.device.index])
            else:
                dist.barrier()

    # ------------------------------------------------------------------------------------------ cuda plumbing
    def _setup_cuda(self) -> None:
        from ..ops import cuda as K

        self.K = K
        f = self.fabric
        assert self.alloc is not None, "the CUDA backend needs the flat buffers in symmetric memory"
        self.ctrl = SymmetricBuffer(f, CTRL_BYTES)
        self.stats_buf = SymmetricBuffer(f, max(self.n_stats, 4) * 4)
        self.stats = self.stats_buf.tensor(torch.float32, max(self.n_stats, 4))
        self.stat_ptrs = self.stats_buf.ptr_array()
        self.partials = [self.ctrl.tensor(torch.float32, 1, PARTIAL_OFF + 64 * i) for i in range(2)]
        self.partial_ptrs = [self.ctrl.ptr_array(PARTIAL_OFF + 64 * i) for i in range(2)]
        self.slot_ptrs = [self.ctrl.ptr_array(SLOT_BYTES * s) for s in range(MAX_BUCKETS + 2)]
        bufs = self.alloc.buffers
        self.grad_ptrs = [bufs[(i, "grad")].ptr_array() for i in range(len(self.groups))]
        self.shadow_ptrs = [bufs[(i, "shadow")].ptr_array() for i in range(len(self.groups))]
        self.master_ptrs = [bufs[(i, "master")].ptr_array() if (i, "master") in bufs else None
                            for i in range(len(self.groups))]
        self.own_shadow_ptrs = [(C.c_void_p * 1)(bufs[(i, "shadow")].own) for i in range(len(self.groups))]
        self.side = torch.cuda.Stream(device=f.device, priority=-1)    # its few CTAs go first when an SM frees up
        self.gather_stream = torch.cuda.Stream(device=f.device)
        self.err = K.err_word(f.device)

    def _side_barrier(self) -> None:
        """Barrier of the deferred phase: its own flag slot and epoch counter, launched on the side stream."""
        K = self.K
        self.defer_epoch += 1
        K._check(K.lib.b200_barrier_sum(self.slot_ptrs[MAX_BUCKETS + 1], self.rank, self.world,
                                        C.c_uint(self.defer_epoch), self.timeout_ms, None, 0, None,
                                        C.c_void_p(self.err.data_ptr()), C.c_void_p(self.side.cuda_stream)), "barrier")

    def on_forward(self, name: str) -> None:
        """Called by the model's forward pass before it touches the weights of phase ``name`` ("core", "coda")."""
        ev = self.deferred_events.pop(name, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)

    def finish_deferred(self) -> None:
        """Every reader of parameters other than the model's forward pass: wait for the deferred updates."""
        for name in list(self.deferred_events):
            self.on_forward(name)

    def _barrier(self, sum_into=None, partial_index: int = 0) -> None:
        K = self.K
        self.epoch += 1
        K._check(K.lib.b200_barrier_sum(self.slot_ptrs[0], self.rank, self.world, C.c_uint(self.epoch), self.timeout_ms,
                                        self.partial_ptrs[partial_index] if sum_into is not None else None,
                                        1 if sum_into is not None else 0,
                                        C.c_void_p(sum_into.data_ptr() if sum_into is not None else 0),
                                        C.c_void_p(self.err.data_ptr()), C.c_void_p(K._stream())), "barrier")

    # ------------------------------------------------------------------------------------------ per step
    def timeline(self) -> dict:
        """Milliseconds relative to the start of the last traced step (B200_TRACE=1): when each bucket's reduce-scatter
        started and ended on the side stream, when the backward pass ended on the main stream, and when the step
        ended.  A bucket whose interval lies before ``backward_end`` ran under the backward pass."""
        tr = self.trace
        if not tr or "start" not in tr:
            return {}
        torch.cuda.synchronize(self.fabric.device)
        t0 = tr["start"]
        out = {"backward_end": round(t0.elapsed_time(tr["backward_end"]), 2),
               "step_end": round(t0.elapsed_time(tr["step_end"]), 2), "buckets": {}}
        for name, (a, b, ctas) in tr.get("buckets", {}).items():
            out["buckets"][name] = {"start": round(t0.elapsed_time(a), 2), "end": round(t0.elapsed_time(b), 2),
                                    "ctas": ctas or 296}
        for name, (a, b, ctas) in tr.get("deferred", {}).items():   # update + push that ran beside the next forward
            out.setdefault("deferred_update", {})[name] = {"start": round(t0.elapsed_time(a), 2),
                                                           "end": round(t0.elapsed_time(b), 2), "ctas": ctas}
        return out

    def begin_step(self, model, accumulating: bool) -> None:
        """Before the forward pass: (zero3) start pulling the other ranks' new parameter pieces; arm the model's
        phase hooks when this micro-batch ends an accumulation window."""
        if self.tracing and self.backend == "cuda" and not accumulating:
            self.trace = {"start": torch.cuda.Event(enable_timing=True)}
            self.trace["start"].record()
        if self.zero3 and self.dirty and self.backend == "cuda":
            self._launch_gathers()
        if model is not None:
            model._phase_cb = self.on_phase if (not accumulating and self.overlap and self.world > 1) else None
            model._fwd_cb = self.on_forward if self.defer else None
        elif self.defer:
            self.finish_deferred()

    def on_phase(self, name: str) -> None:
        """Called from a tensor hook during backward: the gradients of bucket ``name`` are complete on this rank."""
        if name in self.buckets:
            self._fire(name, 0 if name in self.full_width else self.overlap_ctas)

    def _fix_unwritten(self, b: _Bucket) -> None:
        """Gradient buffers are not cleared between steps (the first contribution of a window stores); a tensor that
        received nothing in this window must read as zero."""
        for p in b.params:
            if not getattr(p, "_fused_grad", False):
                continue
            w = getattr(p, "_written", 3)
            if w == 3:
                continue
            if w == 0 or p.dim() != 2:
                p.grad.zero_()
            else:
                half = p.shape[1] // 2
                if not w & 1:
                    p.grad[:, :half].zero_()
                if not w & 2:
                    p.grad[:, half:].zero_()
            p._written = 3

    def _fire(self, name: str, ctas: int) -> None:
        b = self.buckets[name]
        if b.fired:
            return
        b.fired = True
        with nvtx.range(f"reduce-scatter:{name}"):
            self._fire_now(b, ctas)

    def _fire_now(self, b: _Bucket, ctas: int) -> None:
        self._fix_unwritten(b)
        if self.backend != "cuda" or self.world == 1:
            return
        K = self.K
        epoch = C.c_uint(self.reduce_count + 1)
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        # The "my gradients of this bucket are complete" signal is issued by the first CTA of the reduce-scatter kernel
        # itself, never by a launch of its own: a separate signal kernel can be starved by this GPU's own waiting
        # reduce-scatter CTAs while the peer waits for it (every rank then sits out the wait limit).  All ranks fire
        # their buckets in the same order (hooks in graph order, the rest in the same completion order), so waiting for the peers'
        # kernels of the same bucket to start cannot cycle.
        self.side.wait_event(ev)
        if self.tracing:
            t0 = torch.cuda.Event(enable_timing=True)
            t0.record(self.side)
        partial = self.partials[self.reduce_count & 1]
        first = True
        for gi, tb in b.tables:
            K._check(K.lib.b200_rs_table(self.grad_ptrs[gi], self.rank, self.world, C.byref(tb),
                                         C.c_void_p(partial.data_ptr()), self.slot_ptrs[b.slot],
                                         epoch if first else C.c_uint(0), 1, self.timeout_ms, ctas,
                                         C.c_void_p(self.err.data_ptr()), C.c_void_p(self.side.cuda_stream)),
                     "rs_table")
            first = False
        if self.tracing:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record(self.side)
            self.trace.setdefault("buckets", {})[b.name] = (t0, t1, ctas)

    def step(self, optimizer, max_norm: float, grad_scale: float, do_update: bool) -> None:
        """After the backward pass of the last micro-batch of a window: finish the reduction, clip, update."""
        if self.tracing and self.backend == "cuda" and "start" in self.trace:
            self.trace["backward_end"] = torch.cuda.Event(enable_timing=True)
            self.trace["backward_end"].record()
        for name in self.order:
            self._fire(name, 0)
        if self.backend == "cuda":
            self._step_cuda(optimizer, max_norm, grad_scale, do_update)
        else:
            self._step_torch(optimizer, max_norm, grad_scale, do_update)
        if self.tracing and self.backend == "cuda" and "start" in self.trace:
            self.trace["step_end"] = torch.cuda.Event(enable_timing=True)
            self.trace["step_end"].record()
        for b in self.buckets.values():
            b.fired = False
        self.reduce_count += 1
        if self.zero3 and do_update:
            self.dirty = True

    # ------------------------------------------------------------------------------------------ cuda step
    def _launch_tables(self):
        for name in self.order:
            for gi, tb in self.buckets[name].tables:
                yield gi, tb

    def _step_cuda(self, optimizer, max_norm, grad_scale, do_update) -> None:
        K = self.K
        st = C.c_void_p(K._stream())
        gn = C.c_void_p(optimizer.gnorm_sq.data_ptr())
        pi = self.reduce_count & 1
        if self.world > 1:
            done = torch.cuda.Event()
            done.record(self.side)
            torch.cuda.current_stream().wait_event(done)
            self._barrier(sum_into=optimizer.gnorm_sq, partial_index=pi)
            if os.environ.get("B200_DEBUG_NORM") == "1" and not bool(torch.isfinite(optimizer.gnorm_sq).all()):
                self._report_nonfinite(pi)
        else:
            optimizer.compute_grad_norm_sq()
        first_update = optimizer.step_count == 0
        if do_update:
            optimizer.step_count += 1
            args = []
            for gi, h in enumerate(optimizer.param_groups):
                push_master = (gi == len(self.groups) - 1) and self.world > 1   # the fp32-consumed norm/bias group
                n_push = 1 if (self.zero3 and not push_master) else self.world
                args.append(_opt_args(optimizer, h, max_norm=max_norm, grad_scale=grad_scale, first_update=first_update,
                                      n_push=n_push, push_master=push_master,
                                      master_sharded=self.master_sharded[gi], n_ranks=self.world))
            if optimizer.update_clipping:
                self.stats.zero_()
                for gi, tb in self._launch_tables():
                    g = self.groups[gi]
                    K._check(K.lib.b200_opt_stats(C.c_void_p(g.grad.data_ptr()), C.c_void_p(g.state["v"].data_ptr()),
                                                  C.byref(tb), self.rank, gn, C.byref(args[gi]),
                                                  C.c_void_p(self.stats.data_ptr()), st), "opt_stats")
                if self.world > 1:
                    self._barrier()
            def launch(gi, tb, a, stream):
                g = self.groups[gi]
                shadows = self.own_shadow_ptrs[gi] if a.n_push == 1 and self.world > 1 else self.shadow_ptrs[gi]
                K._check(K.lib.b200_opt_table(
                    C.c_void_p(g.master.data_ptr()), C.c_void_p(g.grad.data_ptr()), C.c_void_p(g.state["m"].data_ptr()),
                    C.c_void_p(g.state["v"].data_ptr()), shadows, self.master_ptrs[gi] if a.push_master else None,
                    self.stat_ptrs, C.byref(tb), self.rank, gn, C.byref(a), stream), "opt_table")

            later = {"core": [], "coda": []}
            for name in self.order:
                phase = name.split(".")[0]
                for gi, tb in self.buckets[name].tables:
                    if self.defer and phase in later and not args[gi].push_master:
                        later[phase].append((gi, tb))
                    else:
                        launch(gi, tb, args[gi], st)
            if self.defer and (later["core"] or later["coda"]):
                self._launch_deferred(later, args, launch)
        if self.world > 1:
            self.partials[1 - pi].zero_()
            self._barrier()

    def _launch_deferred(self, later: dict, args: list, launch) -> None:
        """Update + push of the core and coda weights on the side stream, after everything the main stream has issued
        so far (the norm is known, the immediate part of the update owns the link first).  Each phase ends with a
        cross-rank barrier of its own and an event the next forward pass waits on."""
        self.finish_deferred()                      # a step that came without a forward pass in between
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self.side.wait_event(ev)
        side = C.c_void_p(self.side.cuda_stream)
        for phase in ("core", "coda"):
            if self.tracing:
                t0 = torch.cuda.Event(enable_timing=True)
                t0.record(self.side)
            for gi, tb in later[phase]:
                a = OptArgsC.from_buffer_copy(args[gi])
                a.max_ctas = self.defer_ctas[phase]
                launch(gi, tb, a, side)
            self._side_barrier()
            done = torch.cuda.Event(enable_timing=self.tracing)
            done.record(self.side)
            self.deferred_events[phase] = done
            if self.tracing:
                self.trace.setdefault("deferred", {})[phase] = (t0, done, self.defer_ctas[phase])

    def _report_nonfinite(self, pi: int) -> None:
        """Debug aid (B200_DEBUG_NORM=1): which of this rank's reduced pieces are not finite."""
        bad = []
        for gi, g in enumerate(self.groups):
            for t in range(len(g.params)):
                s, n = self.plans[gi].segment(t, self.rank)
                if n and not bool(torch.isfinite(g.grad[s:s + n]).all()):
                    bad.append(g.names[t])
        print(f"[rank {self.rank}] non-finite norm at reduce {self.reduce_count}: own partial "
              f"{float(self.partials[pi])}, status {int(self.err)}, non-finite pieces {bad[:8]} ({len(bad)} total)",
              flush=True)

    # ------------------------------------------------------------------------------------------ zero3 gathers
    def _launch_gathers(self) -> None:
        """Pull the other ranks' updated bf16 pieces into the local full-size copies, bucket by bucket in the order
        the forward pass needs them, on a side stream.  Row-sharded QKV / gate-up weights are left to the first GEMM
        that uses them (``AgHandle``)."""
        K = self.K
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        self.gather_stream.wait_event(ev)
        st = C.c_void_p(self.gather_stream.cuda_stream)
        for name in self.gather_order:
            b = self.buckets[name]
            for gi, ids in b.tensors.items():
                g, plan = self.groups[gi], self.plans[gi]
                pull = []
                for t in ids:
                    h = getattr(g.params[t], "_ag", None)
                    if h is not None and h.usable:
                        h.pending = True
                    else:
                        pull.append(t)
                if gi == len(self.groups) - 1:
                    continue          # the fp32 group is pushed by the update kernel in every mode
                for tb in plan.tables(pull, self.rank):
                    K._check(K.lib.b200_ag_table(self.shadow_ptrs[gi], self.rank, self.world, C.byref(tb), 64, st),
                             "ag_table")
            b.gather_event = torch.cuda.Event()
            b.gather_event.record(self.gather_stream)
            for p in b.params:
                p._gather_wait = b
        self.dirty = False

    @torch.no_grad()
    def reduce_check(self) -> float:
        """Diagnostic (collective): sums the gradients now in the local buffers twice -- NCCL all-reduce on copies and
        the bucket kernels in place -- and returns the largest relative difference over this rank's pieces."""
        assert self.backend == "cuda" and self.world > 1
        self.finish_deferred()
        copies = [g.grad.clone() for g in self.groups]
        for c in copies:
            dist.all_reduce(c)
        for name in self.order:
            self._fire(name, 0)
        done = torch.cuda.Event()
        done.record(self.side)
        torch.cuda.current_stream().wait_event(done)
        self._barrier()
        worst = 0.0
        self.last_check = []
        for gi, (g, c) in enumerate(zip(self.groups, copies)):
            for t in range(len(g.params)):
                s, n = self.plans[gi].segment(t, self.rank)
                if n:
                    ref_n = float(c[s:s + n].norm())
                    d = float((g.grad[s:s + n] - c[s:s + n]).norm()) / (ref_n + 1e-30)
                    if d > 1e-5:
                        self.last_check.append((g.names[t], d, float(g.grad[s:s + n].norm()), ref_n))
                    worst = max(worst, d)
        self.partials[self.reduce_count & 1].zero_()
        self._barrier()
        for b in self.buckets.values():
            b.fired = False
        self.reduce_count += 1
        return worst

    def replicas_identical(self) -> bool:
        """Collective: do all ranks hold bit-identical bf16 compute copies?"""
        self.sync_parameters()
        sums = torch.stack([g.shadow.view(torch.int16).to(torch.int32).sum(dtype=torch.int64) for g in self.groups
                            if g.shadow is not None]).to(torch.float64)
        lo, hi = sums.clone(), sums.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return bool(torch.equal(lo, hi))

    def sync_parameters(self) -> None:
        """Make the local bf16 copies complete now (parameter-sharded mode; before validation, export or comparison).
        Every rank must call it at the same point: the owners' pieces must not change while peers read them."""
        self.finish_deferred()
        if not (self.zero3 and self.dirty and self.backend == "cuda"):
            return
        self._launch_gathers()
        main = torch.cuda.current_stream()
        for b in self.buckets.values():
            for p in b.params:
                h = getattr(p, "_ag", None)
                if h is not None and h.pending:
                    h.pull_now()
                p._gather_wait = None
            if b.gather_event is not None:
                main.wait_event(b.gather_event)

    # ------------------------------------------------------------------------------------------ torch backend
    @torch.no_grad()
    def _step_torch(self, optimizer, max_norm, grad_scale, do_update) -> None:
        """Same bookkeeping with torch.distributed collectives; every rank updates only its own pieces."""
        multi = self.world > 1 and dist.is_initialized()
        part = torch.zeros(1, dtype=torch.float32, device=self.groups[0].grad.device)
        for gi, g in enumerate(self.groups):
            if multi:
                dist.all_reduce(g.grad)
            for t in range(len(g.params)):
                s, n = self.plans[gi].segment(t, self.rank)
                part += g.grad[s:s + n].float().pow(2).sum()
        if multi:
            dist.all_reduce(part)
        optimizer.gnorm_sq.copy_(part)
        gn = float(part.sqrt()) * grad_scale
        first_update = optimizer.step_count == 0
        if do_update and math.isfinite(gn):
            optimizer.step_count += 1
            clip = min(1.0, max_norm / (gn + 1e-6)) if max_norm > 0 else 1.0
            gs = grad_scale * clip
            stats = torch.zeros(self.n_stats, dtype=torch.float32)
            if optimizer.update_clipping:
                for gi, (g, h) in enumerate(zip(self.groups, optimizer.param_groups)):
                    soff = self.plans[gi].state_offsets(self.rank)
                    for t in range(len(g.params)):
                        s, n = self.plans[gi].segment(t, self.rank)
                        if n:
                            stats[self.stat_base[gi] + t] = optimizer.clip_stat(
                                g.grad[s:s + n], g.state["v"][soff[t]:soff[t] + n], h, gs, first_update)
                if multi:
                    dist.all_reduce(stats)
            for gi, (g, h) in enumerate(zip(self.groups, optimizer.param_groups)):
                soff = self.plans[gi].state_offsets(self.rank)
                sharded = self.master_sharded[gi]
                for t in range(len(g.params)):
                    s, n = self.plans[gi].segment(t, self.rank)
                    if not n:
                        continue
                    so = soff[t]
                    pm = g.master[so:so + n] if sharded else g.master[s:s + n]
                    stat = float(stats[self.stat_base[gi] + t]) / self.plans[gi].numels[t] \
                        if optimizer.update_clipping else None
                    optimizer.update_piece(pm, g.grad[s:s + n], g.state["m"][so:so + n], g.state["v"][so:so + n], h,
                                           optimizer.step_count, gs, first_update, stat)
                    if g.shadow is not None:
                        g.shadow[s:s + n].copy_(pm)
            if multi:
                self._exchange_torch()
        for g in self.groups:
            g.grad.zero_()

    def _exchange_torch(self) -> None:
        """Owners broadcast their new pieces (bf16 copies; fp32 masters where they are replicated)."""
        for gi, g in enumerate(self.groups):
            plan = self.plans[gi]
            for t in range(len(g.params)):
                for q in range(self.world):
                    s, n = plan.segment(t, q)
                    if not n:
                        continue
                    if g.shadow is not None:
                        piece = g.shadow[s:s + n].float()
                        dist.broadcast(piece, src=q)
                        g.shadow[s:s + n].copy_(piece)
                    if not self.master_sharded[gi]:
                        dist.broadcast(g.master[s:s + n], src=q)

    # ------------------------------------------------------------------------------------------ checkpoint helpers
    @torch.no_grad()
    def gather_master(self) -> None:
        """Make every rank's replicated fp32 master copies complete (owners broadcast their pieces)."""
        self.finish_deferred()
        if self.world == 1 or not dist.is_initialized():
            return
        for gi, g in enumerate(self.groups):
            if self.master_sharded[gi]:
                continue
            plan = self.plans[gi]
            for t in range(len(g.params)):
                for q in range(self.world):
                    s, n = plan.segment(t, q)
                    if n:
                        dist.broadcast(g.master[s:s + n], src=q)

    @torch.no_grad()
    def full_master(self, gi: int, t: int) -> torch.Tensor:
        """fp32 values of one whole tensor (collective when the group's masters are sharded)."""
        g, plan = self.groups[gi], self.plans[gi]
        shape = g.params[t].shape
        if not self.master_sharded[gi]:
            return g.master[g.offsets[t]:g.offsets[t] + plan.numels[t]].view(shape)
        soff = plan.state_offsets(self.rank)
        per = plan.pers[t]
        mine = torch.zeros(per, dtype=torch.float32, device=g.master.device)
        n = plan.segment(t, self.rank)[1]
        mine[:n].copy_(g.master[soff[t]:soff[t] + n])
        if self.world > 1 and dist.is_initialized():
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine)
        else:
            parts = [mine]
        return torch.cat(parts)[:plan.numels[t]].view(shape)

    @torch.no_grad()
    def load_full_master(self, gi: int, t: int, value: torch.Tensor) -> None:
        """Inverse of ``full_master`` for this rank's piece (and the local bf16 copy of the whole tensor)."""
        g, plan = self.groups[gi], self.plans[gi]
        flat = value.reshape(-1).to(device=g.master.device, dtype=torch.float32)
        if self.master_sharded[gi]:
            lo, hi = plan.local(t, self.rank)
            so = plan.state_offsets(self.rank)[t]
            g.master[so:so + hi - lo].copy_(flat[lo:hi])
        else:
            g.master[g.offsets[t]:g.offsets[t] + plan.numels[t]].copy_(flat)
        if g.shadow is not None:
            g.shadow[g.offsets[t]:g.offsets[t] + plan.numels[t]].copy_(flat)

    def persistent_bytes(self) -> dict:
        """Bytes this rank holds for parameters, gradients and optimizer state, by kind."""
        out = {"master": 0, "grad": 0, "shadow": 0, "moments": 0}
        for g in self.groups:
            out["master"] += g.master.numel() * 4
            out["grad"] += g.grad.numel() * 4
            out["shadow"] += g.shadow.numel() * 2 if g.shadow is not None else 0
            out["moments"] += (g.state["m"].numel() + g.state["v"].numel()) * 4
        return out

    def close(self) -> None:
        if self.backend != "cuda":
            return
        torch.cuda.synchronize(self.fabric.device)
        self.ctrl.close()
        self.stats_buf.close()
        for buf in self.alloc.buffers.values():
            buf.close()


P2PReducer = ShardedStepper   # older name


class AgHandle:
    """First-use gather of one row-sharded weight in the parameter-sharded mode: the first GEMM of a step that
    multiplies by the weight pulls the other ranks' rows while it computes (``b200_ag_gemm``)."""

    def __init__(self, stepper: ShardedStepper, gi: int, t: int):
        from ..ops import cuda as K

        self.K = K
        g, plan = stepper.groups[gi], stepper.plans[gi]
        self.stepper = stepper
        self.where = (gi, t)
        self.N, self.Kdim = g.params[t].shape
        self.rows_per = plan.rows_per_rank(t)
        self.usable = self.rows_per is not None and self.Kdim % 8 == 0 and stepper.world <= 8
        self.pending = False
        off_bytes = g.offsets[t] * 2
        buf = stepper.alloc.buffers[(gi, "shadow")]
        if self.usable:
            row_bytes = self.Kdim * 2
            self.shard_ptrs = (C.c_void_p * stepper.world)(
                *[p + off_bytes + q * self.rows_per * row_bytes for q, p in enumerate(buf.ptrs)])
        self.full_ptr = buf.own + off_bytes
        self.done = torch.zeros((self.N + 239) // 240 + 1, dtype=torch.int32, device=stepper.fabric.device)
        self._ag = K._sig("b200_ag_gemm", [C.c_void_p] * 5 + [C.c_int] * 9 + [C.c_void_p, C.c_void_p])

    def gemm(self, x2: torch.Tensor) -> torch.Tensor | None:
        """y = x2 W^T while gathering W; None when the input is not eligible (the caller then waits for a plain pull)."""
        if not (self.pending and self.usable) or x2.shape[0] < 256 or x2.dtype != torch.bfloat16 or x2.stride(1) != 1:
            return None
        K, s = self.K, self.stepper
        y = torch.empty(x2.shape[0], self.N, dtype=torch.bfloat16, device=x2.device)
        K._check(self._ag(x2.data_ptr(), C.cast(self.shard_ptrs, C.c_void_p), self.full_ptr, y.data_ptr(),
                          self.done.data_ptr(), x2.shape[0], self.N, self.Kdim, x2.stride(0), self.N, s.world, s.rank,
                          self.rows_per, 0, K._stream(), K.err_word(x2.device).data_ptr()), "ag_gemm")
        self.pending = False
        return y

    def pull_now(self) -> None:
        """Plain pull of this weight (its first use was not a GEMM that can gather)."""
        if not self.pending:
            return
        K, s = self.K, self.stepper
        gi, t = self.where
        for tb in s.plans[gi].tables([t], s.rank):
            K._check(K.lib.b200_ag_table(s.shadow_ptrs[gi], s.rank, s.world, C.byref(tb), 0, C.c_void_p(K._stream())),
                     "ag_table")
        self.pending = False
