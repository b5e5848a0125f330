"""ELLISAdam: the AdamW variant of the reference's production runs (recpre/optim.py:728-1035).

Options (all off by default, the Frontier run enables update_clipping, atan_adam, running_init, decouple_wd):
nesterov momentum, eps adjustment (eps inside the root), per-tensor update clipping ``lr / max(1, rms(g^2 / v))``,
Kahan-compensated parameter updates, low-precision moment buffers, ``running_init`` (moments start at the first
gradient), tensor-wise finite check / gradient normalisation, Adafactor-like beta schedules, atan2 update
``p -= step * atan2(m, sqrt(v) / sqrt(bc2))``, decoupled weight decay relative to the constructor lr, a brute-force
update-norm clip, and a polynomial-EMA beta2.  ``lr`` may be a tensor that the training loop rewrites every step.
"""
from __future__ import annotations

import copy
from math import sqrt
from typing import Optional

import torch
from torch.optim import Optimizer


class ELLISAdam(Optimizer):
    def __init__(self, params, lr=3e-4, betas=(0.9, 0.99), eps: float = 1e-6, weight_decay: float = 1e-2, *,
                 foreach=None, nesterov=False, eps_adjustment=False, update_clipping=False,
                 kahan_sum_compensation=False, buffer_dtype=None, running_init=False, tensor_wise_finite_check=False,
                 tensor_wise_gradient_normalization=False, adafactor_like_beta_corrections=False, atan_adam=False,
                 decouple_wd=True, brute_force_clip: Optional[float] = None, poly_ema_p: Optional[float] = None):
        if isinstance(buffer_dtype, str):
            buffer_dtype = getattr(torch, buffer_dtype)
        defaults = dict(lr=torch.tensor(float(lr), dtype=torch.float32), init_lr=copy.deepcopy(float(lr)),
                        betas=tuple(betas), eps=eps, weight_decay=weight_decay, nesterov=nesterov,
                        eps_adjustment=eps_adjustment, update_clipping=update_clipping,
                        kahan_sum_compensation=kahan_sum_compensation, buffer_dtype=buffer_dtype,
                        running_init=running_init, tensor_wise_finite_check=tensor_wise_finite_check,
                        tensor_wise_gradient_normalization=tensor_wise_gradient_normalization,
                        adafactor_like_beta_corrections=adafactor_like_beta_corrections, atan_adam=atan_adam,
                        decouple_wd=decouple_wd, brute_force_clip=brute_force_clip, poly_ema_p=poly_ema_p)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            lr, init_lr, wd, eps = group["lr"], group["init_lr"], group["weight_decay"], group["eps"]
            lr_f = float(lr)
            first = True
            for p in group["params"]:
                if p.grad is None:
                    continue
                bdt = group["buffer_dtype"] or p.dtype
                g = p.grad.to(bdt)
                if group["tensor_wise_finite_check"] and not bool(torch.isfinite(g).all()):
                    continue
                if group["tensor_wise_gradient_normalization"]:
                    g = g / g.norm()
                st = self.state[p]
                if not st:
                    st["step"] = torch.tensor(0.0)
                    if group["running_init"]:
                        st["exp_avg"], st["exp_avg_sq"] = g.clone(), g.pow(2)
                    else:
                        st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(g), torch.zeros_like(g)
                    st["kahan_comp"] = torch.zeros_like(p) if group["kahan_sum_compensation"] else None
                m, v, t = st["exp_avg"], st["exp_avg_sq"], st["step"]
                beta1, beta2 = b1, b2
                if group["adafactor_like_beta_corrections"]:
                    if first:
                        t += 1
                    tt = float(t)
                    beta1 = (b1 ** tt - b1) / (b1 ** tt - 1) if tt > 1 else 0.0
                    beta2 = (b2 ** tt - b2) / (b2 ** tt - 1) if tt > 1 else 0.0
                if group["poly_ema_p"] is not None:
                    tt = float(t)
                    beta2 = tt / (tt + group["poly_ema_p"])
                first = False
                if group["nesterov"]:
                    m.lerp_(g, 2 * (1 - beta1) - (1 - beta1) ** 2)
                else:
                    m.lerp_(g, 1 - beta1)
                v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
                step_size = lr_f
                if group["update_clipping"]:
                    rms = g.pow(2).div_(v.clamp_(min=eps ** 2)).mean().sqrt()
                    step_size = step_size / float(rms.clamp(min=1.0))
                if not group["adafactor_like_beta_corrections"]:
                    t += 1
                    tt = float(t)
                    bc2 = 1 - beta2 ** tt
                    step_size = step_size / (1 - beta1 ** tt)
                else:
                    bc2 = 1.0
                bc2_sqrt = sqrt(bc2)
                decay = 1 - (lr_f / init_lr * wd if group["decouple_wd"] else lr_f * wd)
                if group["atan_adam"]:
                    update = torch.atan2(m, v.sqrt().div_(bc2_sqrt))
                elif group["eps_adjustment"]:
                    update = m / v.div(bc2).add_(eps ** 2).sqrt()
                else:
                    update = m / v.sqrt().div_(bc2_sqrt).add_(eps)
                if group["brute_force_clip"] is not None:
                    update = update / torch.clamp(update.norm(), min=group["brute_force_clip"])
                if group["kahan_sum_compensation"]:
                    comp = st["kahan_comp"]
                    comp.mul_(decay).add_(update.to(comp.dtype), alpha=-step_size)
                    old = p.detach().clone()
                    p.add_(comp)
                    comp.add_(old.sub_(p))
                else:
                    p.mul_(decay).add_(update.to(p.dtype), alpha=-step_size)
                if group["nesterov"]:
                    m.lerp_(g, 1 - 1 / beta1)
        return loss
