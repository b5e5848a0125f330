"""Smaller research optimizers selectable by name: LionW (recpre/optim.py:266-375), SophiaG (:415-626) and
OrthogonalNesterov with a quintic Newton-Schulz orthogonalisation (:1762-1858)."""
from __future__ import annotations

import torch
from torch.optim import Optimizer


class LionW(Optimizer):
    """Sign-momentum optimizer with decoupled weight decay: p -= lr * sign(b1 m + (1-b1) g); m = b2 m + (1-b2) g."""

    def __init__(self, params, lr: float = 1e-4, betas=(0.9, 0.99), weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            lr = float(group["lr"])
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p)
                m = st["exp_avg"]
                p.mul_(1 - lr * group["weight_decay"])
                p.add_(torch.sign(m.mul(b1).add_(p.grad, alpha=1 - b1)), alpha=-lr)
                m.mul_(b2).add_(p.grad, alpha=1 - b2)
        return loss


class SophiaG(Optimizer):
    """Sophia with a Gauss-Newton-Bartlett Hessian estimate: p -= lr * clip(m / max(rho * bs * h, eps), 1).
    ``update_hessian()`` is called by the training loop every k steps after a backward pass on sampled labels."""

    def __init__(self, params, lr: float = 1e-4, betas=(0.965, 0.99), rho: float = 0.04, weight_decay: float = 0.1,
                 bs: int = 1):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), rho=rho, weight_decay=weight_decay))
        self.bs = bs

    @torch.no_grad()
    def update_hessian(self):
        for group in self.param_groups:
            _, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "hessian" not in st:
                    st["exp_avg"], st["hessian"] = torch.zeros_like(p), torch.zeros_like(p)
                st["hessian"].mul_(b2).addcmul_(p.grad, p.grad, value=1 - b2)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, _ = group["betas"]
            lr = float(group["lr"])
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "hessian" not in st:
                    st["exp_avg"], st["hessian"] = torch.zeros_like(p), torch.zeros_like(p)
                m, h = st["exp_avg"], st["hessian"]
                m.mul_(b1).add_(p.grad, alpha=1 - b1)
                p.mul_(1 - lr * group["weight_decay"])
                ratio = (m.abs() / (group["rho"] * self.bs * h + 1e-15)).clamp(max=1)
                p.addcmul_(m.sign(), ratio, value=-lr)
        return loss


def zeroth_power_via_newtonschulz5(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Approximate orthogonalisation of a matrix by five quintic Newton-Schulz iterations in bf16."""
    a, b, c = 3.4445, -4.7750, 2.0315
    X = G.bfloat16() / (G.norm() + eps)
    transposed = G.size(0) > G.size(1)
    if transposed:
        X = X.T
    for _ in range(steps):
        A = X @ X.T
        B = A @ X
        X = a * X + b * B + c * A @ B
    return (X.T if transposed else X).to(G.dtype)


class OrthogonalNesterov(Optimizer):
    """Nesterov momentum whose 2-D updates are orthogonalised (Muon-style)."""

    def __init__(self, params, lr: float = 0.02, momentum: float = 0.9, nesterov: bool = True, steps: int = 5,
                 weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, steps=steps,
                                      weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            lr = float(group["lr"])
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(g)
                buf = st["momentum_buffer"]
                buf.mul_(group["momentum"]).add_(g)
                g = g.add(buf, alpha=group["momentum"]) if group["nesterov"] else buf
                if g.ndim == 2:
                    g = zeroth_power_via_newtonschulz5(g, steps=group["steps"])
                    g = g * max(g.size(0), g.size(1)) ** 0.5
                if group["weight_decay"]:
                    p.mul_(1 - lr * group["weight_decay"])
                p.add_(g.to(p.dtype), alpha=-lr)
        return loss
