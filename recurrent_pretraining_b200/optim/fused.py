"""Fused flat-buffer AdamW for the GPU path.

One kernel launch per optimizer group does: global-norm clip (factor derived on the device from the reduced
squared norm), decoupled weight decay, both moment updates, the parameter update in fp32, the bf16 compute
copy, and zeroing of the gradient buffer.  No host synchronisation: a non-finite norm turns the launch into a
no-op on the device (train.py:446-461 of the reference skips such steps on the host).
Semantics are those of ``torch.optim.AdamW`` (recpre/optim.py:115-120) or, with ``atan2=True``, the
atan2 update of the reference's ELLISAdam without its per-tensor options (recpre/optim.py:1008-1019).
"""
from __future__ import annotations

import torch

from ..ops import reference as ref


class FusedAdamW:
    def __init__(self, flat_groups, lr=4e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, atan2=False):
        self.groups = flat_groups
        self.defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        self.atan2 = atan2
        self.step_count = 0
        self.param_groups = []
        for g in flat_groups:
            h = dict(self.defaults)
            h.update(g.hyper)
            h["params"] = g.params
            self.param_groups.append(h)
            g.state["m"] = torch.zeros_like(g.master)
            g.state["v"] = torch.zeros_like(g.master)
            g.state["range"] = (0, g.numel)
        dev = flat_groups[0].master.device
        self.gnorm_sq = torch.zeros(1, dtype=torch.float32, device=dev)

    def shard(self, ranges) -> None:
        """Keep optimizer state only for ``ranges[i] = (lo, hi)`` of group i (sharded data-parallel update)."""
        for g, (lo, hi) in zip(self.groups, ranges):
            dev = g.master.device
            g.state["m"] = torch.zeros(max(hi - lo, 4), dtype=torch.float32, device=dev)
            g.state["v"] = torch.zeros(max(hi - lo, 4), dtype=torch.float32, device=dev)
            g.state["range"] = (lo, hi)

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

    # -- step ------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, max_norm: float = 0.0, grad_scale: float = 1.0, zero_grad: bool = True, norm_ready: bool = False):
        """Update all groups.  ``gnorm_sq`` must hold the squared norm of the *stored* gradients (before
        ``grad_scale``) unless clipping is off; it is computed here when ``norm_ready`` is False."""
        if not norm_ready:
            self.compute_grad_norm_sq()
        self.step_count += 1
        for g, h in zip(self.groups, self.param_groups):
            lr = float(h["lr"])
            b1, b2 = h["betas"]
            if g.master.is_cuda:
                from ..ops import cuda as C

                C.adamw_(g.master, g.grad, g.state["m"], g.state["v"], g.shadow, self.gnorm_sq, lr=lr, beta1=b1,
                         beta2=b2, eps=h["eps"], wd=h["weight_decay"], step=self.step_count, max_norm=max_norm,
                         grad_scale=grad_scale, zero_grad=zero_grad, atan2=self.atan2)
            else:
                gn = self.gnorm_sq.sqrt() * grad_scale
                if not torch.isfinite(gn):
                    if zero_grad:
                        g.grad.zero_()
                    continue
                clip = min(1.0, max_norm / (float(gn) + 1e-6)) if max_norm > 0 else 1.0
                ref.adamw_step(g.master, g.grad, g.state["m"], g.state["v"], lr, b1, b2, h["eps"], h["weight_decay"],
                               self.step_count, grad_scale * clip)
                if g.shadow is not None:
                    g.shadow.copy_(g.master)
                if zero_grad:
                    g.grad.zero_()

    def grad_norm(self, grad_scale: float = 1.0) -> torch.Tensor:
        return self.gnorm_sq.sqrt() * grad_scale

    def zero_grad(self, set_to_none: bool = False):
        for g in self.groups:
            g.grad.zero_()

    def state_dict(self):
        return {"step": self.step_count,
                "groups": [{"m": g.state["m"], "v": g.state["v"], "range": g.state["range"], "names": g.names,
                            "offsets": g.offsets,
                            "hyper": {k: v for k, v in h.items() if k != "params"}}
                           for g, h in zip(self.groups, self.param_groups)]}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for g, h, s in zip(self.groups, self.param_groups, sd["groups"]):
            g.state["m"].copy_(s["m"])
            g.state["v"].copy_(s["v"])
            for k, v in s.get("hyper", {}).items():
                h[k] = v
