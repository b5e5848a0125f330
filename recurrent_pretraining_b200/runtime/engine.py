"""Training engine: one object that owns the model, the flat parameter store, the optimizer and the gradient
synchronisation, and exposes ``train_step(input_ids, labels)``.

Step semantics follow the reference (train.py:389-475, recpre/utils.py:1196-1206): gradients of
``grad_accum`` micro-batches are summed locally, then summed across ranks and divided by the world size,
clipped by global L2 norm, and applied; the very first optimizer step of a run only clears the gradients
(``skip_first_step``); a non-finite norm skips the update.

Two execution modes:
* ``fused`` (CUDA): bf16 compute copies + fp32 master weights in flat buffers; wgrad GEMMs write into the flat
  fp32 gradient buffer (the first contribution of an accumulation window stores, later ones accumulate, so the
  buffer is never cleared); the 1/(accum*world) scale and the clip factor are folded into the fused update
  kernel (AdamW, or the ELLISAdam flags of the reference's production run), so no host synchronisation happens
  inside a step.  With several GPUs the reduction is bucketed and overlapped with the backward pass
  (``parallel/p2p.py``).
* ``torch`` (CPU or any ``torch.optim`` optimizer): conventional loss scaling, ``clip_grad_norm_`` and
  ``optimizer.step()``; used for the gloo plumbing tests and the research optimizers.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..optim.fused import FusedAdamW
from ..utils import nvtx
from ..optim.groups import get_param_groups
from ..parallel.flat import flatten_group


class TrainEngine:
    def __init__(self, model, fabric=None, *, lr: float = 4e-4, weight_decay: float = 0.1, betas=(0.9, 0.95),
                 eps: float = 1e-8, grad_clip: float = 1.0, grad_accum: int = 1, skip_first_step: bool = True,
                 no_weight_decay_for_bias_and_norm_params: bool = False, optimizer: Optional[object] = None,
                 mode: Optional[str] = None, atan2: bool = False, lr_fn=None, allow_skip_nonfinite: bool = True,
                 update_clipping: bool = False, running_init: bool = False, decouple_wd: bool = False):
        from ..parallel.fabric import Fabric

        self.fabric = fabric if fabric is not None else Fabric.single(next(model.parameters()).device)
        self.model = model
        self.device = self.fabric.device
        self.grad_clip, self.grad_accum = grad_clip, max(int(grad_accum), 1)
        self.skip_first_step = skip_first_step
        self.micro_step = 0
        self.window_base = 0          # micro-step at which accumulation windows are anchored (moves on resume)
        self.optimizer_step = 0
        self.lr_fn = lr_fn
        self.base_lr = lr
        self.last_grad_norm = None
        self.mode = mode or ("fused" if self.device.type == "cuda" and optimizer is None else "torch")
        model.to(self.device)
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        groups = get_param_groups(named, no_weight_decay_for_bias_and_norm_params, with_names=True)
        self.flat_groups = []
        if self.mode == "fused":
            shard_masters = getattr(self.fabric, "shards_masters", False)
            for gi, g in enumerate(groups):
                hyper = {"lr": lr * g["base_lr"], "base_lr": g["base_lr"],
                         "weight_decay": g.get("weight_decay", weight_decay)}
                # the small fp32 group (norm scales, biases) is read in fp32 by the kernels and stays replicated
                shard = (self.fabric.world_size, self.fabric.global_rank) if shard_masters and gi < len(groups) - 1 \
                    else None
                self.flat_groups.append(flatten_group(g["params"], g["names"], self.device, True, hyper,
                                                      alloc=self.fabric.buffer_allocator(gi), shard=shard))
            self.optimizer = FusedAdamW(self.flat_groups, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                        atan2=atan2, update_clipping=update_clipping, running_init=running_init,
                                        decouple_wd=decouple_wd)
            self.fabric.register_flat_groups(self.flat_groups, model, self.optimizer)
            self._fused_params = [p for g in self.flat_groups for p in g.params if getattr(p, "_fused_grad", False)]
            if not self.fabric.is_distributed:
                # one GPU: the core / coda part of the update runs beside the next forward pass (optim/fused.py)
                self.optimizer.enable_deferred(model)
        else:
            if optimizer is None:
                for g in groups:
                    g.pop("names", None)
                    g.setdefault("weight_decay", weight_decay)
                optimizer = torch.optim.AdamW(groups, lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
            for g in optimizer.param_groups:
                g.setdefault("base_lr", 1.0)
            self.optimizer = optimizer
            self.ddp = None
            if getattr(self.fabric, "grad_sync", "") == "ddp" and self.fabric.is_distributed:
                # the reference's alternative to its hand-rolled all-reduce: torch DistributedDataParallel with unused-
                # parameter detection, needed because of the untracked recurrences (recpre/utils.py:1154-1155,
                # finetuning_simple_example.py:176-179)
                from torch.nn.parallel import DistributedDataParallel as DDP

                ids = [self.device.index] if self.device.type == "cuda" else None
                self.ddp = DDP(model, device_ids=ids, find_unused_parameters=True, gradient_as_bucket_view=True)
        self.params = [p for _, p in named]

    # ------------------------------------------------------------------------------------------
    def set_lr(self, lr: float) -> None:
        for h in self.optimizer.param_groups:
            h["lr"] = lr * h.get("base_lr", 1.0)

    def is_accumulating(self) -> bool:
        return (self.micro_step - self.window_base) % self.grad_accum != 0

    def train_step(self, input_ids: torch.Tensor, labels: torch.Tensor, **fwd_kwargs) -> dict:
        """One micro-batch: forward, backward, and -- on accumulation boundaries -- reduce, clip, update.
        Returns ``{"loss": device tensor, "grad_norm": device tensor or None, "depths": (n, k)}``."""
        model = self.model
        model.train()
        self.micro_step += 1
        model.step = self.micro_step
        accumulating = self.is_accumulating()
        if self.mode == "fused":
            if (self.micro_step - 1 - self.window_base) % self.grad_accum == 0:
                self._begin_window()
            self.fabric.begin_backward(model, accumulating)
        ddp = getattr(self, "ddp", None)
        if ddp is not None:
            import contextlib

            ctx = ddp.no_sync() if accumulating else contextlib.nullcontext()
            with ctx:
                with nvtx.range("forward"):
                    out = ddp(input_ids, labels=labels, **fwd_kwargs)
                loss = out["loss"]
                with nvtx.range("backward"):
                    (loss / self.grad_accum).backward()      # DDP averages over ranks inside backward
        else:
            with nvtx.range("forward"):
                out = model(input_ids, labels=labels, **fwd_kwargs)
            loss = out["loss"]
            with nvtx.range("backward"):
                if self.mode == "fused":
                    loss.backward()
                else:
                    (loss / self.grad_accum).backward()
        result = {"loss": loss.detach(), "log_ppl": out["log_ppl"], "grad_norm": None,
                  "depths": getattr(model, "last_depths", (0, 0))}
        if accumulating:
            return result
        if self.lr_fn is not None:
            self.set_lr(self.lr_fn(self.micro_step))
        do_update = not (self.skip_first_step and self.optimizer_step == 0)
        if self.mode == "fused":
            world = self.fabric.world_size
            scale = 1.0 / (self.grad_accum * world)
            with nvtx.range("reduce+update"):
                fused_done = self.fabric.fused_reduce_and_step(self.optimizer, self.grad_clip, scale, do_update)
            if fused_done:
                result["grad_norm"] = self.optimizer.grad_norm(scale)
                self.last_grad_norm = result["grad_norm"]
                self.optimizer_step += 1
                return result
            self._finish_window()
            norm_ready = self.fabric.reduce_gradients(self.optimizer)  # sum over ranks
            if do_update:
                self.optimizer.step(max_norm=self.grad_clip, grad_scale=scale, zero_grad=False, norm_ready=norm_ready)
            elif not norm_ready:
                self.optimizer.compute_grad_norm_sq()
            result["grad_norm"] = self.optimizer.grad_norm(scale)
        else:
            if getattr(self, "ddp", None) is None:
                self.fabric.all_reduce_gradients(self.params)
            gn = torch.nn.utils.clip_grad_norm_(self.params, self.grad_clip if self.grad_clip > 0 else math.inf)
            finite = bool(torch.isfinite(gn))
            if do_update and finite:
                self.optimizer.step()
            self.optimizer.zero_grad(set_to_none=False)
            result["grad_norm"] = gn
        self.last_grad_norm = result["grad_norm"]
        self.optimizer_step += 1
        return result

    def _begin_window(self) -> None:
        """Start of an accumulation window.  A gradient that the kernels write themselves (weight-gradient GEMMs,
        embedding and head backward; known from ``_gemm_written`` once it happened) is marked unwritten, so its first
        contribution stores.  Every other gradient is accumulated by autograd and is cleared here (norm scales, biases:
        a few hundred KB)."""
        deferred = getattr(self.optimizer, "defer_ranges", None) or {}
        st = self._stepper()
        if st is not None and getattr(st, "defer", False):
            deferred = dict.fromkeys(range(len(self.flat_groups) - 1))     # every group but the fp32 one
        for gi, g in enumerate(self.flat_groups):
            fused = [p for p in g.params if getattr(p, "_fused_grad", False)]
            if fused and not any(getattr(p, "_gemm_written", False) for p in fused):
                if gi in deferred:
                    self._finish_deferred()             # the late part of the last update still reads these gradients
                g.grad.zero_()                      # one launch for a whole group of autograd-accumulated gradients
                for p in fused:
                    p._written = 3
                continue
            for p in fused:
                if getattr(p, "_gemm_written", False):
                    p._written = 0
                else:
                    if gi in deferred:
                        self._finish_deferred()
                    p.grad.zero_()
                    p._written = 3

    def _finish_deferred(self) -> None:
        st = self._stepper()
        if st is not None:
            st.finish_deferred()
        if hasattr(self.optimizer, "finish_deferred"):
            self.optimizer.finish_deferred()

    def _finish_window(self) -> None:
        """A tensor that received no gradient in this window must read as zero (nothing else clears the buffers)."""
        for p in self._fused_params:
            if p._written != 3:
                if p._written == 0 or p.dim() != 2:
                    p.grad.zero_()
                else:
                    half = p.shape[1] // 2
                    (p.grad[:, :half] if not p._written & 1 else p.grad[:, half:]).zero_()
                p._written = 3

    @torch.no_grad()
    def eval_loss(self, input_ids, labels, num_steps_pair=None):
        self.fabric.sync_parameters()
        self.model.eval()
        out = self.model(input_ids, labels=labels, num_steps_pair=num_steps_pair)
        self.model.train()
        return out["loss"]

    # ------------------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"micro_step": self.micro_step, "optimizer_step": self.optimizer_step,
                "optimizer": self.optimizer.state_dict()}

    def load_state_dict(self, sd: dict, other_shards=None) -> None:
        """``other_shards``: callable returning the engine state dicts of all ranks of the saved run; needed only when
        the optimizer state has to be re-cut for a different world size."""
        self.micro_step = sd["micro_step"]
        self.optimizer_step = sd["optimizer_step"]
        if isinstance(self.optimizer, FusedAdamW):
            others = (lambda: [o["optimizer"] for o in other_shards()]) if other_shards is not None else None
            self.optimizer.load_state_dict(sd["optimizer"], others)
        else:
            self.optimizer.load_state_dict(sd["optimizer"])
        # a checkpoint taken inside an accumulation window does not carry the partial gradient sums: the window
        # restarts at the resume point
        self.window_base = self.micro_step

    def _stepper(self):
        return getattr(self.fabric, "_p2p", None)

    def _sharded_index(self) -> dict:
        """id(param) -> (group, tensor) for parameters whose fp32 master exists only as per-rank pieces."""
        out = {}
        for gi, g in enumerate(self.flat_groups):
            if getattr(g, "master_sharded", False):
                for t, p in enumerate(g.params):
                    out[id(p)] = (gi, t)
        return out

    @torch.no_grad()
    def model_state_dict(self) -> dict:
        """fp32 state dict of the model on the CPU.  Collective when masters are sharded or partly stale on this rank
        (every rank must call it)."""
        st = self._stepper()
        if st is not None:
            st.gather_master()
        if hasattr(self.optimizer, "finish_deferred"):
            self.optimizer.finish_deferred()
        sharded = self._sharded_index()
        out = {}
        for k, v in self.model.state_dict(keep_vars=True).items():
            if id(v) in sharded:
                out[k] = st.full_master(*sharded[id(v)]).detach().to("cpu", copy=True)
            else:
                out[k] = v.detach().to("cpu", copy=True)
        return out

    @torch.no_grad()
    def load_model_state(self, sd: dict, strict: bool = True) -> None:
        own = self.model.state_dict(keep_vars=True)
        sharded = self._sharded_index()
        st = self._stepper()
        if st is not None:
            st.finish_deferred()
        if hasattr(self.optimizer, "finish_deferred"):
            self.optimizer.finish_deferred()
        for k, v in sd.items():
            if k not in own:
                if strict and k != "lm_head.weight":
                    raise KeyError(f"unexpected key {k} in checkpoint")
                continue
            if id(own[k]) in sharded:
                st.load_full_master(*sharded[id(own[k])], v)
            else:
                own[k].data.copy_(v.to(own[k].dtype)) if torch.is_tensor(own[k]) else None
        missing = [k for k in own if k not in sd and k != "lm_head.weight"]
        if strict and missing:
            raise KeyError(f"missing keys in checkpoint: {missing[:5]}")
        self.refresh_shadows()

    def refresh_shadows(self) -> None:
        """Re-derive the bf16 compute copies from the fp32 masters (after loading a checkpoint)."""
        for g in self.flat_groups:
            if g.shadow is not None and not getattr(g, "master_sharded", False):
                g.shadow.copy_(g.master)
