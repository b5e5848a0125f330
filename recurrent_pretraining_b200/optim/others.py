"""Smaller research optimizers selectable by name: LionW (recpre/optim.py:266-375), SophiaG (:415-626) and
OrthogonalNesterov with a quintic Newton-Schulz orthogonalisation (:1762-1858)."""
from __future__ import annotations

import torch
from torch.optim import Optimizer


class LionW(Optimizer):
    """Sign-momentum optimizer with decoupled weight decay: p -= lr * sign(b1 m + (1-b1) g); m = b2 m + (1-b2) g.
    After every step the cosine between the update and its sign is kept for telemetry
    (``get_post_step_metrics``, recpre/optim.py:291-309); the sums stay on the parameters' device."""

    def __init__(self, params, lr: float = 1e-4, betas=(0.9, 0.99), weight_decay: float = 0.0, **kwargs):
        assert lr > 0.0 and all(0.0 <= b <= 1.0 for b in betas)
        super().__init__(params, dict(lr=lr, betas=tuple(betas), weight_decay=weight_decay))
        for group in self.param_groups:
            group["initial_lr"] = group["lr"]
        self._update_total_dot_prod = self._update_total_norm = self._signed_update_total_norm = None

    def get_post_step_metrics(self, module=None, process_group=None) -> dict:
        """``{"update_cos_sim": <update, sign(update)> / (|update| |sign(update)|)}`` of the last step; with a process
        group the three sums are reduced over it first (sharded parameters)."""
        dot, un, sn = self._update_total_dot_prod, self._update_total_norm, self._signed_update_total_norm
        if dot is None or un is None or sn is None:
            return {}
        if process_group is not None and torch.distributed.is_initialized():
            sq = torch.stack([dot, un ** 2, sn ** 2])
            torch.distributed.all_reduce(sq, group=process_group)
            dot, un, sn = sq[0], sq[1].sqrt(), sq[2].sqrt()
        return {"update_cos_sim": dot / torch.clamp(un * sn, min=1e-8)}

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        dot = un2 = sn2 = None
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
                update = m.mul(b1).add_(p.grad, alpha=1 - b1)
                signed = torch.sign(update)
                p.add_(signed, alpha=-lr)
                m.mul_(b2).add_(p.grad, alpha=1 - b2)
                uf, sf = update.float(), signed.float()
                d, u2, s2 = (uf * sf).sum(), uf.pow(2).sum(), sf.pow(2).sum()
                dot = d if dot is None else dot + d.to(dot.device)
                un2 = u2 if un2 is None else un2 + u2.to(un2.device)
                sn2 = s2 if sn2 is None else sn2 + s2.to(sn2.device)
        if dot is not None:
            self._update_total_dot_prod, self._update_total_norm = dot, un2.sqrt()
            self._signed_update_total_norm = sn2.sqrt()
        return loss


class SophiaG(Optimizer):
    """Sophia with a Gauss-Newton-Bartlett Hessian estimate: p -= lr * clip(|m| / (rho * bs * h + 1e-15), 1) * sign(m)
    after a decoupled weight decay (recpre/optim.py:415-626).  ``update_hessian()`` is called by the training loop every
    k steps after a backward pass on sampled labels."""

    def __init__(self, params, lr: float = 1e-4, betas=(0.965, 0.99), rho: float = 0.04, weight_decay: float = 0.1,
                 bs: int | None = None, *, maximize: bool = False, capturable: bool = False, **kwargs):
        """``bs`` (tokens per step; scales the Hessian estimate) may be fixed here or passed to ``step``; the
        reference's ``step`` defaults it to 5120.  ``maximize`` flips the gradient's sign; ``capturable`` is accepted
        for signature compatibility (nothing here synchronises with the host)."""
        if not lr >= 0.0 or not 0.0 <= betas[0] < 1.0 or not 0.0 <= betas[1] < 1.0 or not rho >= 0.0 \
                or not weight_decay >= 0.0:
            raise ValueError("invalid SophiaG hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=tuple(betas), rho=rho, weight_decay=weight_decay,
                                      maximize=maximize, capturable=capturable))
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
    def step(self, closure=None, bs=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        bs = bs if bs is not None else (self.bs if self.bs is not None else 5120)
        for group in self.param_groups:
            b1, _ = group["betas"]
            lr = float(group["lr"])
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "hessian" not in st:
                    st["exp_avg"], st["hessian"] = torch.zeros_like(p), torch.zeros_like(p)
                st["step"] = st.get("step", 0) + 1
                m, h = st["exp_avg"], st["hessian"]
                g = -p.grad if group.get("maximize", False) else p.grad
                m.mul_(b1).add_(g, alpha=1 - b1)
                p.mul_(1 - lr * group["weight_decay"])
                ratio = (m.abs() / (group["rho"] * bs * h + 1e-15)).clamp(max=1)
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
    """Nesterov momentum whose 2-D updates are orthogonalised by Newton-Schulz iterations; every other parameter -- and
    any matrix with an extent equal to ``vocab_dim`` (embedding, head) -- takes an AdamW step (recpre/optim.py:1762-1832;
    argument names and defaults as there).

    Matrix branch, as in the reference: ``buf = momentum * buf + g``; ``u = NS5(g + momentum * buf)`` (or ``NS5(buf)``
    without nesterov); ``p -= 0.1 * lr * sqrt(numel) / ||u|| * u``.

    AdamW branch: the reference decays the weights and divides its first moment by a bias-corrected denominator, but it
    never accumulates either moment, so those parameters only ever shrink by the weight decay.  Here the moments are
    accumulated (a plain AdamW step with the group's ``betas`` / ``eps``); ``frozen_moments=True`` restores the
    reference's arithmetic for comparisons."""

    def __init__(self, params, lr: float = 4e-4, momentum: float = 0.95, nesterov: bool = True, zeropower_iters: int = 5,
                 eps: float = 1e-5, betas=(0.9, 0.95), weight_decay: float = 1e-5, vocab_dim: int = 32768,
                 frozen_moments: bool = False, steps: int | None = None):
        if steps is not None:                            # older keyword of this package
            zeropower_iters = steps
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, zeropower_iters=zeropower_iters,
                                      eps=eps, betas=tuple(betas), weight_decay=weight_decay, vocab_dim=vocab_dim,
                                      frozen_moments=frozen_moments))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            lr, momentum = float(group["lr"]), group["momentum"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                st = self.state[p]
                if p.ndim == 2 and group["vocab_dim"] not in p.shape:
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = torch.zeros_like(g)
                    buf = st["momentum_buffer"]
                    buf.mul_(momentum).add_(g)
                    g = g.add(buf, alpha=momentum) if group["nesterov"] else buf
                    update = zeroth_power_via_newtonschulz5(g, steps=group["zeropower_iters"])
                    scale = update.numel() ** 0.5 / float(update.norm())
                    p.add_(update.to(p.dtype), alpha=-lr * 0.1 * scale)
                    continue
                if "step" not in st:
                    st["step"] = 0
                    st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(p), torch.zeros_like(p)
                st["step"] += 1
                b1, b2 = group["betas"]
                p.mul_(1 - lr * group["weight_decay"])
                bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                if group["frozen_moments"]:
                    denom = (st["exp_avg"].sqrt() / bc2 ** 0.5).add_(group["eps"])
                else:
                    st["exp_avg"].lerp_(g, 1 - b1)
                    st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                    denom = (st["exp_avg_sq"].sqrt() / bc2 ** 0.5).add_(group["eps"])
                p.addcdiv_(st["exp_avg"], denom, value=-lr / bc1)
        return loss
