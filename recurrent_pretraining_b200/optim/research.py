"""Research optimizers that the reference keeps selectable by name: Lilith, IVON and a blocked, rank-sharded Shampoo
with Adam grafting.

Behavioural counterparts: recpre/optim.py:630-715 (Lilith), :1046-1303 (IVON), :1313-1755 (Shampoo with Adam
grafting, blocks dealt round-robin over ranks, parameters made consistent after the step).  IVON keeps ONE momentum /
Hessian vector per group; Shampoo exchanges the updated blocks with one all-reduce per parameter (each block has
exactly one owner, the other ranks contribute zeros) instead of one broadcast per block.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Optional

import torch
import torch.distributed as dist
from torch.optim import Optimizer


class Lilith(Optimizer):
    """Trust-ratio scaled double-momentum Adam variant (recpre/optim.py:630-715)."""

    def __init__(self, params, lr: float, eps: float = 1e-8, beta1_m: float = 0.9, beta2_m: float = 0.99,
                 beta_v: float = 0.999, weight_decay: float = 0.01, g_norm_min: float = 1e-4, ratio_min: float = 1e-4,
                 acceleration: float = 1, ema_k: int = 0, ema_beta: float = 0.99, **_):
        super().__init__(params, dict(lr=lr, eps=eps, beta1_m=beta1_m, beta2_m=beta2_m, beta_v=beta_v,
                                      weight_decay=weight_decay, g_norm_min=g_norm_min, ratio_min=ratio_min,
                                      acceleration=acceleration, ema_k=ema_k, ema_beta=ema_beta))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            lr = float(g["lr"])
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["m_avg1"] = torch.zeros_like(grad)
                    st["m_avg2"] = torch.zeros_like(grad)
                    st["v_avg"] = torch.zeros_like(grad)
                    if g["ema_k"] > 0:
                        st["ema"] = p.detach().clone()
                st["step"] += 1
                if sum(grad.shape) > 1:  # scalars keep their raw gradient
                    ratio = (p.norm() / grad.norm().clamp(min=g["g_norm_min"])).clamp(min=g["ratio_min"])
                    grad = grad * ratio
                m1, m2, v = st["m_avg1"], st["m_avg2"], st["v_avg"]
                before = m1.clone()
                m1.add_(m2).lerp_(grad, 1 - g["beta1_m"])
                m2.lerp_(m1 - before, 1 - g["beta2_m"])
                u = m1 + g["acceleration"] * m2
                v.lerp_(u.square(), 1 - g["beta_v"])
                u = u / (v / (1 - g["beta_v"] ** st["step"]) + g["eps"]).sqrt()
                u.add_(p, alpha=g["weight_decay"])
                p.add_(u, alpha=-lr)
                if g["ema_k"]:
                    st["ema"].lerp_(p, 1 - g["ema_beta"])
                    if st["step"] % g["ema_k"] == 0:
                        p.copy_(st["ema"])
        return loss


def _running_mean(mean: Optional[torch.Tensor], sample: torch.Tensor, count: int) -> torch.Tensor:
    return sample.clone() if mean is None else mean + (sample - mean) / count


class IVON(Optimizer):
    """Improved variational online Newton (recpre/optim.py:1046-1303).

    Usage per optimizer step: ``for _ in range(mc_samples): with opt.sampled_params(train=True): loss.backward()``
    then ``opt.step()``.  Inside the context the parameters are a draw from the current Gaussian posterior; leaving it
    restores the mean and records the gradient sample (and noise*gradient for the Price estimator).
    """

    hessian_approx_methods = ("price", "gradsq")

    def __init__(self, params, lr: float, ess: float, hess_init: float = 1e-3, beta1: float = 0.9,
                 beta2: float = 1 - 1e-5, weight_decay: float = 1e-6, mc_samples: int = 1, hess_approx: str = "price",
                 clip_radius: float = 1e-3, sync: bool = False, debias: bool = True, rescale_lr: bool = True):
        for name, ok in (("lr", lr > 0), ("mc_samples", mc_samples >= 1), ("weight_decay", weight_decay > 0),
                         ("hess_init", hess_init > 0), ("ess", ess > 0), ("clip_radius", clip_radius > 0),
                         ("beta1", 0 < beta1 < 1), ("beta2", 0 < beta2 < 1),
                         ("hess_approx", hess_approx in self.hessian_approx_methods)):
            if not ok:
                raise ValueError(f"Invalid {name}")
        super().__init__(params, dict(lr=lr, mc_samples=mc_samples, beta1=beta1, beta2=beta2, weight_decay=weight_decay,
                                      hess_init=hess_init, ess=ess, clip_radius=clip_radius))
        self.mc_samples, self.hess_approx, self.sync = mc_samples, hess_approx, sync
        self.debias, self.rescale_lr = debias, rescale_lr
        self.current_step = 0
        plist = [p for g in self.param_groups for p in g["params"]]
        if len({p.device for p in plist}) > 1 or len({p.dtype for p in plist}) > 1:
            raise ValueError("IVON needs all parameters on one device and in one dtype")
        self._device = plist[0].device if plist else torch.device("cpu")
        self._dtype = plist[0].dtype if plist else torch.get_default_dtype()
        for g in self.param_groups:
            g["numel"] = sum(p.numel() for p in g["params"])
            g["momentum"] = torch.zeros(g["numel"], device=self._device, dtype=self._dtype)
            g["hess"] = torch.full((g["numel"],), float(g["hess_init"]), device=self._device, dtype=self._dtype)
        self._numel = sum(g["numel"] for g in self.param_groups)
        self._clear_samples()

    def _clear_samples(self):
        self.state["count"] = 0
        self.state["avg_grad"] = self.state["avg_nxg"] = self.state["avg_gsq"] = None

    def _params(self):
        for g in self.param_groups:
            yield from g["params"]

    @contextmanager
    def sampled_params(self, train: bool = False):
        noise = torch.cat([torch.randn(g["numel"], device=self._device, dtype=self._dtype) /
                           (g["ess"] * (g["hess"] + g["weight_decay"])).sqrt() for g in self.param_groups])
        mean = torch.cat([p.data.flatten() for p in self._params()])
        off = 0
        for p in self._params():
            p.data = (mean[off:off + p.numel()] + noise[off:off + p.numel()]).view(p.shape)
            off += p.numel()
        try:
            yield
        finally:
            off, grads = 0, []
            for p in self._params():
                p.data = mean[off:off + p.numel()].view(p.shape)
                off += p.numel()
                if train:
                    grads.append(p.grad.flatten() if p.grad is not None else torch.zeros(p.numel(), device=self._device,
                                                                                       dtype=self._dtype))
            if train:
                gs = torch.cat(grads)
                n = self.state["count"] = self.state["count"] + 1
                self.state["avg_grad"] = _running_mean(self.state["avg_grad"], gs, n)
                if self.hess_approx == "price":
                    self.state["avg_nxg"] = _running_mean(self.state["avg_nxg"], noise * gs, n)
                else:
                    self.state["avg_gsq"] = _running_mean(self.state["avg_gsq"], gs.square(), n)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            losses = []
            for _ in range(self.mc_samples):
                with torch.enable_grad():
                    losses.append(closure())
            loss = sum(losses) / self.mc_samples
        if self.sync and dist.is_available() and dist.is_initialized():
            for key in ("avg_grad", "avg_nxg", "avg_gsq"):
                if self.state[key] is not None:
                    dist.all_reduce(self.state[key])
                    self.state[key].div_(dist.get_world_size())
        self.current_step += 1
        off = 0
        for g in self.param_groups:
            sl = slice(off, off + g["numel"])
            b1, b2, wd = g["beta1"], g["beta2"], g["weight_decay"]
            g["momentum"] = b1 * g["momentum"] + (1 - b1) * self.state["avg_grad"][sl]
            h = g["hess"]
            if self.hess_approx == "price":
                f = self.state["avg_nxg"][sl] * (h + wd) * g["ess"]
            else:
                f = self.state["avg_gsq"][sl] * g["ess"]
            g["hess"] = b2 * h + (1 - b2) * f + 0.5 * (1 - b2) ** 2 * (h - f).square() / (h + wd)
            lr = float(g["lr"]) * (g["hess_init"] + wd) if self.rescale_lr else float(g["lr"])
            debias = 1.0 - b1 ** float(self.current_step) if self.debias else 1.0
            mean = torch.cat([p.data.flatten() for p in g["params"]])
            mean = mean - lr * torch.clip((g["momentum"] / debias + wd * mean) / (g["hess"] + wd), -g["clip_radius"],
                                          g["clip_radius"])
            o = 0
            for p in g["params"]:
                p.data = mean[o:o + p.numel()].view(p.shape)
                o += p.numel()
            off += g["numel"]
        self._clear_samples()
        return loss


class ZeroShampooWithAdamGraftingOptimizer(Optimizer):
    """Blocked Shampoo whose update is rescaled to the Frobenius norm of the Adam direction (grafting).

    Every parameter is viewed as a matrix [prod(shape[:-1]), shape[-1]] and cut into ``block_size`` squares; block i
    (global counter over all parameters) is owned by rank ``i % world``; after the step every parameter is summed over
    ranks so that all replicas agree (recpre/optim.py:1413-1425,1472-1556,1641-1665).  Gradients are expected to be
    averaged already.
    """

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), shampoo_eps=1e-6, adam_betas=(0.9, 0.999), adam_eps=1e-8,
                 precondition_frequency=None, start_preconditioning=4, independent_weight_decay=True,
                 weight_decay=1e-3, block_size=128, **_):
        super().__init__(params, dict(lr=lr, betas=betas, shampoo_eps=shampoo_eps, adam_betas=adam_betas,
                                      adam_eps=adam_eps,
                                      precondition_frequency=precondition_frequency or start_preconditioning,
                                      start_preconditioning=start_preconditioning,
                                      independent_weight_decay=independent_weight_decay, weight_decay=weight_decay))
        self.block_size = block_size
        self.distributed = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank() if self.distributed else 0
        self.world_size = dist.get_world_size() if self.distributed else 1
        self._plan = []  # (param, group, [(r0, r1, c0, c1), ...]) owned by this rank
        counter = 0
        for g in self.param_groups:
            for p in g["params"]:
                rows, cols = self._matrix_shape(p)
                mine = []
                for r0 in range(0, rows, block_size):
                    for c0 in range(0, cols, block_size):
                        if counter % self.world_size == self.rank:
                            mine.append((r0, min(r0 + block_size, rows), c0, min(c0 + block_size, cols)))
                        counter += 1
                self._plan.append((p, g, mine))
        self.num_blocks = counter

    @staticmethod
    def _matrix_shape(p):
        return (p.shape[0], 1) if p.ndim == 1 else (int(p.numel() // p.shape[-1]), p.shape[-1])

    @staticmethod
    def _inv_fourth_root(mats: torch.Tensor) -> torch.Tensor:
        evals, evecs = torch.linalg.eigh(mats.float())
        evals = evals.clamp(min=1e-12).pow(-0.25)
        return ((evecs * evals.unsqueeze(-2)) @ evecs.transpose(-1, -2)).to(mats.dtype)

    def _block_state(self, p, key, block, eps):
        st = self.state[p].setdefault("blocks", {})
        if key not in st:
            st[key] = dict(step=0, m=torch.zeros_like(block), v=torch.zeros_like(block),
                           L=eps * torch.eye(block.shape[0], device=block.device, dtype=block.dtype),
                           R=eps * torch.eye(block.shape[1], device=block.device, dtype=block.dtype), PL=None, PR=None)
        return st[key]

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for p, g, mine in self._plan:
            if p.grad is None:
                continue
            rows, cols = self._matrix_shape(p)
            P, G = p.data.view(rows, cols), p.grad.view(rows, cols)
            lr = float(g["lr"])
            b1 = g["betas"][0]
            ab1, ab2 = g["adam_betas"]
            if self.world_size > 1:
                keep = torch.zeros_like(P, dtype=torch.bool)
            for (r0, r1, c0, c1) in mine:
                blk, grad = P[r0:r1, c0:c1], G[r0:r1, c0:c1]
                st = self._block_state(p, (r0, c0), blk, g["shampoo_eps"])
                st["step"] += 1
                if g["independent_weight_decay"]:
                    blk.mul_(1 - lr * g["weight_decay"])
                st["L"].mul_(b1).add_(grad @ grad.t(), alpha=1 - b1)
                st["R"].mul_(b1).add_(grad.t() @ grad, alpha=1 - b1)
                st["m"].mul_(ab1).add_(grad, alpha=1 - ab1)
                st["v"].mul_(ab2).addcmul_(grad, grad, value=1 - ab2)
                adam_dir = (st["m"] / (1 - ab1 ** st["step"])) / ((st["v"] / (1 - ab2 ** st["step"])).sqrt() +
                                                                    g["adam_eps"])
                if st["step"] >= g["start_preconditioning"]:
                    if st["step"] % g["precondition_frequency"] == 0 or st["PL"] is None:
                        st["PL"], st["PR"] = self._inv_fourth_root(st["L"]), self._inv_fourth_root(st["R"])
                    sh = st["PL"] @ st["m"] @ st["PR"]
                    update = torch.linalg.norm(adam_dir) * sh / torch.linalg.norm(sh).clamp(min=1e-30)
                else:
                    update = adam_dir
                blk.add_(update, alpha=-lr)
                if self.world_size > 1:
                    keep[r0:r1, c0:c1] = True
            if self.world_size > 1:  # every block has exactly one owner: zero the rest and sum
                P.mul_(keep)
        if self.world_size > 1:
            for p, _, _ in self._plan:
                if p.grad is not None:
                    dist.all_reduce(p.data)
        return loss
