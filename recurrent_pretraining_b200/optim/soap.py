"""SOAP: Adam in the eigenbasis of Shampoo's preconditioners (recpre/soap.py:34-446, arXiv 2409.11321).

Per 2-D parameter: accumulate ``L = E[G G^T]`` and ``R = E[G^T G]`` for every dimension not larger than
``max_precond_dim`` (so the 15840/17920/35840/65536-wide sides of the flagship stay un-preconditioned), keep their
eigenvectors ``Q_L, Q_R`` (``eigh`` at the first step, one power-iteration + QR refresh every ``precondition_frequency``
steps), run Adam on the rotated gradient ``Q_L^T G Q_R`` and rotate the update back.  The first step only initialises
the preconditioners.

The products are fp32 x fp32: Gram matrices ``G^T G``, the three rotations per step and the power iteration.  On the
flagship they are ~150 TFLOP per optimizer step, seconds as fp32 SIMT GEMMs.  On CUDA tensors with tensor-core
friendly extents they run as three bf16 tcgen05 GEMMs each with fp32 accumulation on split operands
(``ops/cuda.py: matmul_f32``, ~2^-16 relative error); ``eigh`` and ``qr`` stay on the library.  ``B200_SOAP_TENSOR_CORES=0``
keeps ``torch.tensordot``.
"""
from __future__ import annotations

import os

import torch
from torch.optim import Optimizer

_TC = os.environ.get("B200_SOAP_TENSOR_CORES", "1") == "1"


def _contract_first(x: torch.Tensor, mat: torch.Tensor, back: bool) -> torch.Tensor:
    """``tensordot(x, mat, dims=[[0], [1 if back else 0]])`` for 2-D operands: x^T mat (x^T mat^T when ``back``)."""
    if _TC and x.dim() == 2 and x.is_cuda:
        from ..ops import cuda as C

        if C.matmul_f32_supported(x, mat):
            return C.matmul_f32(x, mat, a_mn=True, b_mn=not back)
    return torch.tensordot(x, mat, dims=[[0], [1 if back else 0]])


def _gram(g: torch.Tensor, keep: int) -> torch.Tensor:
    """Sum over every dimension but ``keep`` of the outer product of g with itself."""
    if _TC and g.dim() == 2 and g.is_cuda:
        from ..ops import cuda as C

        if C.matmul_f32_supported(g, g):
            return C.matmul_f32(g, g) if keep == 0 else C.matmul_f32(g, g, a_mn=True, b_mn=True)
    dims = [j for j in range(g.dim()) if j != keep]
    return torch.tensordot(g, g, dims=[dims, dims])


def _mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if _TC and a.is_cuda:
        from ..ops import cuda as C

        if C.matmul_f32_supported(a, b):
            return C.matmul_f32(a, b, b_mn=True)
    return a @ b


class SOAP(Optimizer):
    def __init__(self, params, lr: float = 3e-3, betas=(0.9, 0.95), shampoo_beta: float = -1, eps: float = 1e-8,
                 weight_decay: float = 0.01, precondition_frequency: int = 10, max_precond_dim: int = 10000,
                 merge_dims: bool = False, precondition_1d: bool = False, data_format: str = "channels_first",
                 correct_bias: bool = True):
        assert data_format in ("channels_first", "channels_last")
        self._data_format = data_format       # 4-D weights stored NHWC are merged in NCHW order (recpre/soap.py:96-103)
        defaults = dict(lr=lr, betas=tuple(betas), shampoo_beta=shampoo_beta, eps=eps, weight_decay=weight_decay,
                        precondition_frequency=precondition_frequency, max_precond_dim=max_precond_dim,
                        merge_dims=merge_dims, precondition_1d=precondition_1d, correct_bias=correct_bias)
        super().__init__(params, defaults)

    @staticmethod
    def _merge(shape, max_dim):
        out, cur = [], 1
        for s in shape:
            if cur * s > max_dim:
                if cur > 1:
                    out.append(cur)
                    cur = s
                else:
                    out.append(s)
                    cur = 1
            else:
                cur *= s
        if cur > 1 or not out:
            out.append(cur)
        return out

    def _init_precond(self, g, st, group):
        st["GG"], st["Q"] = [], None
        if g.dim() == 1 and (not group["precondition_1d"] or g.shape[0] > group["max_precond_dim"]):
            st["GG"].append([])
        else:
            for s in g.shape:
                st["GG"].append([] if s > group["max_precond_dim"] else torch.zeros(s, s, device=g.device))
        st["shampoo_beta"] = group["shampoo_beta"] if group["shampoo_beta"] >= 0 else group["betas"][1]

    @staticmethod
    def _project(g, Q, back=False):
        for mat in Q:
            if len(mat) > 0:
                g = _contract_first(g, mat, back)
            else:
                g = g.permute(list(range(1, g.dim())) + [0])
        return g

    def _update_gg(self, g, st):
        beta = st["shampoo_beta"]
        for i, m in enumerate(st["GG"]):
            if len(m) > 0:
                m.lerp_(_gram(g, i), 1 - beta)

    @staticmethod
    def _eigh_basis(mats):
        out = []
        for m in mats:
            if len(m) == 0:
                out.append([])
                continue
            try:
                _, q = torch.linalg.eigh(m.float() + 1e-30 * torch.eye(m.shape[0], device=m.device))
            except Exception:
                _, q = torch.linalg.eigh(m.double() + 1e-30 * torch.eye(m.shape[0], device=m.device, dtype=torch.float64))
                q = q.float()
            out.append(torch.flip(q, [1]))
        return out

    def _refresh_basis(self, st):
        exp_avg_sq = st["exp_avg_sq"]
        new_q = []
        for i, (m, q) in enumerate(zip(st["GG"], st["Q"])):
            if len(m) == 0:
                new_q.append([])
                continue
            mq = _mm(m, q)
            est = (q * mq).sum(0)              # diag(q^T m q)
            order = torch.argsort(est, descending=True)
            exp_avg_sq = exp_avg_sq.index_select(i, order)
            power = mq[:, order]               # m @ q[:, order]
            q_new, _ = torch.linalg.qr(power)
            new_q.append(q_new)
        st["exp_avg_sq"] = exp_avg_sq
        st["Q"] = new_q

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                st = self.state[p]
                shape = g.shape
                nhwc = group["merge_dims"] and g.dim() == 4 and self._data_format == "channels_last"
                if nhwc:
                    g = g.permute(0, 3, 1, 2).contiguous()
                    shape = g.shape
                if group["merge_dims"] and g.dim() > 1:
                    g = g.reshape(self._merge(g.shape, group["max_precond_dim"]))
                if "step" not in st:
                    st["step"] = 0
                    st["exp_avg"], st["exp_avg_sq"] = torch.zeros_like(g), torch.zeros_like(g)
                    self._init_precond(g, st, group)
                    self._update_gg(g, st)
                    st["Q"] = self._eigh_basis(st["GG"])
                    continue  # the first step only initialises the preconditioner
                st["step"] += 1
                gp = self._project(g, st["Q"])
                m, v = st["exp_avg"], st["exp_avg_sq"]
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(gp, gp, value=1 - b2)
                denom = v.sqrt().add_(group["eps"])
                mp = self._project(m, st["Q"])
                step_size = group["lr"]
                if group["correct_bias"]:
                    step_size = step_size * ((1 - b2 ** st["step"]) ** 0.5) / (1 - b1 ** st["step"])
                upd = self._project(mp / denom, st["Q"], back=True)
                upd = upd.reshape(shape)
                if nhwc:
                    upd = upd.permute(0, 2, 3, 1)
                p.add_(upd.to(p.dtype), alpha=-float(step_size))
                if group["weight_decay"] > 0:
                    p.add_(p, alpha=-float(group["lr"]) * group["weight_decay"])
                self._update_gg(g, st)
                if st["step"] % group["precondition_frequency"] == 0:
                    self._refresh_basis(st)
        return loss
