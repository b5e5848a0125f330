"""Differentiable front end of the op set.

CPU tensors take the plain PyTorch statements in ``reference`` (ordinary autograd).  CUDA
tensors take ``torch.autograd.Function``s whose forward and backward launch the sm_100a
kernels through ``ops.cuda``; there is no silent fallback on a GPU: if the native library
is missing the import of ``ops.cuda`` raises.

Weight gradients on the CUDA path go straight into a persistent fp32 gradient buffer from the
wgrad GEMM epilogue: a parameter that carries ``_fused_grad = True`` and a preallocated ``.grad``
gets ``grad (+)= dy^T x`` in place and autograd sees ``None``.  The buffers are never cleared between
optimizer steps: ``param._written`` (bit 0: first half of the columns, bit 1: second half; reset at the
start of every accumulation window by the training engine) tells whether a contribution stores or
accumulates, which saves one read and one write of every gradient per step.

In the parameter-sharded mode a weight may carry ``_ag`` (gathered by its first GEMM of a step) and
``_gather_wait`` (a side-stream pull that the first use has to wait for).
"""
from __future__ import annotations

import math

import torch

from . import reference as ref
from . import sac

_cuda = None


def cuda_backend():
    global _cuda
    if _cuda is None:
        from . import cuda as _c

        _cuda = _c
    return _cuda


def _sync_gather(weight: torch.Tensor) -> None:
    """Parameter-sharded mode: make sure the local bf16 copy of ``weight`` holds this step's values."""
    h = getattr(weight, "_ag", None)
    if h is not None and h.pending:
        h.pull_now()
    b = getattr(weight, "_gather_wait", None)
    if b is not None:
        torch.cuda.current_stream().wait_event(b.gather_event)
        weight._gather_wait = None


def _lp(weight: torch.Tensor) -> torch.Tensor:
    """bf16 compute copy of a parameter: the persistent shadow kept by the optimizer when present."""
    lp = getattr(weight, "_lp", None)
    if lp is not None:
        if hasattr(weight, "_gather_wait"):
            _sync_gather(weight)
        return lp
    return weight if weight.dtype == torch.bfloat16 else weight.detach().to(torch.bfloat16)


def _ag_pending(weight: torch.Tensor) -> bool:
    h = getattr(weight, "_ag", None)
    return h is not None and h.pending


def _gemm_nt_w(x2: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x2 W^T through the weight's bf16 copy; the first use of a row-sharded weight in a step gathers it inside the
    GEMM kernel."""
    h = getattr(weight, "_ag", None)
    if h is not None and h.pending:
        y = h.gemm(x2)
        if y is not None:
            return y
    return cuda_backend().gemm_nt(x2, _lp(weight))


def _store_first(weight: torch.Tensor, mask: int = 3) -> bool:
    """True when this is the first contribution of the accumulation window to the column halves in ``mask``
    (the caller then stores instead of accumulating)."""
    w = getattr(weight, "_written", 3)
    weight._written = w | mask
    weight._gemm_written = True
    return (w & mask) == 0


def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor):
    """dW = dy2^T x2.  Returns the tensor for autograd, or None after writing into the fused gradient buffer."""
    C = cuda_backend()
    if getattr(weight, "_fused_grad", False) and weight.grad is not None:
        C.gemm_tn(dy2, x2, out=weight.grad, accumulate=not _store_first(weight))
        return None
    return C.gemm_tn(dy2, x2, out_dtype=torch.float32).to(weight.dtype)


# ------------------------------------------------------------------------------------------
# linear / adapter
# ------------------------------------------------------------------------------------------
class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        C = cuda_backend()
        x2 = x.reshape(-1, x.shape[-1])
        (y,) = sac.run_op("mm", lambda: (_gemm_nt_w(x2, weight),))
        ctx.save_for_backward(x2, weight)
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        C = cuda_backend()
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = C.gemm_nn(dy2, _lp(weight)).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw = _wgrad(dy2, x2, weight) if ctx.needs_input_grad[1] else None
        return dx, dw


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if x.is_cuda:
        return _Linear.apply(x, weight)
    return ref.linear(x, weight)


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for W = [Wg; Wu] in ONE GEMM whose epilogue applies the gate (forward only: the
    pre-activation is never written, so this is for no-grad passes such as the untracked recurrences and inference)."""
    assert not (torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad))
    if x.is_cuda and _ag_pending(weight):
        return swiglu(linear(x, weight))     # the gathering GEMM has the plain epilogue; once per step
    if x.is_cuda:
        C = cuda_backend()
        x2 = x.reshape(-1, x.shape[-1])
        y = C.gemm(x2, _lp(weight), out_mode=C.OUT_SWIGLU)
        return y.view(*x.shape[:-1], weight.shape[0] // 2)
    return ref.swiglu(ref.linear(x, weight))


class _GatedMLP(torch.autograd.Function):
    """proj(silu(x Wg^T) * (x Wu^T)) for fc = [Wg; Wu] with both elementwise stages inside GEMM epilogues: the gate-up
    GEMM stores the gated product and the pre-activation; in backward the down projection's input-gradient GEMM applies
    the gate's derivative in its epilogue.  Four GEMMs forward + backward pairs, no standalone SwiGLU kernels."""

    @staticmethod
    def forward(ctx, x, w_fc, w_proj):
        C = cuda_backend()
        x2 = x.reshape(-1, x.shape[-1])
        y, h = sac.run_op("mm", lambda: C.linear_swiglu_save(x2, _lp(w_fc)))
        (out,) = sac.run_op("mm", lambda: (C.gemm_nt(y, _lp(w_proj)),))
        ctx.save_for_backward(x2, w_fc, w_proj, h, y)
        ctx.xshape = x.shape
        return out.view(*x.shape[:-1], w_proj.shape[0])

    @staticmethod
    def backward(ctx, dout):
        C = cuda_backend()
        x2, w_fc, w_proj, h, y = ctx.saved_tensors
        d2 = dout.reshape(-1, dout.shape[-1])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dh = C.dswiglu_dgrad(d2, _lp(w_proj), h)
        dw_proj = _wgrad(d2, y, w_proj) if ctx.needs_input_grad[2] else None
        dx = C.gemm_nn(dh, _lp(w_fc)).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw_fc = _wgrad(dh, x2, w_fc) if ctx.needs_input_grad[1] else None
        return dx, dw_fc, dw_proj


def gated_mlp(x: torch.Tensor, w_fc: torch.Tensor, w_proj: torch.Tensor) -> torch.Tensor:
    """SwiGLU MLP without biases; the GPU path with gradients fuses both elementwise stages into GEMM epilogues."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.numel() // x.shape[-1] >= 128 and not _ag_pending(w_fc) \
            and (w_fc.shape[0] // 2) % 8 == 0:
        return _GatedMLP.apply(x, w_fc, w_proj)
    return linear(swiglu(linear(x, w_fc)), w_proj)


class _Adapter(torch.autograd.Function):
    """y = x Ws^T + e We^T with W = [Ws | We] (no concatenation is materialised)."""

    @staticmethod
    def forward(ctx, x, e, weight):
        C = cuda_backend()
        E = x.shape[-1]
        x2, e2 = x.reshape(-1, E), e.reshape(-1, E)
        w = _lp(weight)
        (y,) = sac.run_op("mm", lambda: (C.gemm_nt(x2, w, a2=e2),))  # K loop: x then e against the two halves of W
        ctx.save_for_backward(x2, e2, weight)
        ctx.xshape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        C = cuda_backend()
        x2, e2, weight = ctx.saved_tensors
        E = x2.shape[-1]
        w = _lp(weight)
        dy2 = dy.reshape(-1, E)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = C.gemm_nn(dy2, w[:, :E]).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        de = C.gemm_nn(dy2, w[:, E:]).view(ctx.xshape) if ctx.needs_input_grad[1] else None
        dw = None
        if ctx.needs_input_grad[2]:
            if getattr(weight, "_fused_grad", False) and weight.grad is not None:
                C.gemm_tn(dy2, x2, out=weight.grad[:, :E], accumulate=not _store_first(weight, 1))
                C.gemm_tn(dy2, e2, out=weight.grad[:, E:], accumulate=not _store_first(weight, 2))
            else:
                dw = torch.empty(weight.shape, dtype=torch.float32, device=dy.device)
                C.gemm_tn(dy2, x2, out=dw[:, :E])
                C.gemm_tn(dy2, e2, out=dw[:, E:])
                dw = dw.to(weight.dtype)
        return dx, de, dw


def _half_wgrad(dy2, a2, weight, cols: slice):
    """Gradient of one column half of the adapter weight; fused accumulation when the flat gradient buffer exists."""
    C = cuda_backend()
    if getattr(weight, "_fused_grad", False) and weight.grad is not None:
        mask = 1 if cols.start == 0 else 2
        C.gemm_tn(dy2, a2, out=weight.grad[:, cols], accumulate=not _store_first(weight, mask))
        return None
    dw = torch.zeros(weight.shape, dtype=torch.float32, device=dy2.device)
    C.gemm_tn(dy2, a2, out=dw[:, cols])
    return dw.to(weight.dtype)


class _AdapterInject(torch.autograd.Function):
    """inj = e We^T, the loop-invariant half of the adapter (W = [Ws | We]): computed once per forward pass instead of
    once per recurrence, and its two backward GEMMs run once on the summed gradient."""

    @staticmethod
    def forward(ctx, e, weight):
        C = cuda_backend()
        E = e.shape[-1]
        e2 = e.reshape(-1, E)
        ctx.save_for_backward(e2, weight)
        ctx.eshape = e.shape
        (y,) = sac.run_op("mm", lambda: (C.gemm_nt(e2, _lp(weight)[:, E:]),))
        return y.view(e.shape)

    @staticmethod
    def backward(ctx, dinj):
        C = cuda_backend()
        e2, weight = ctx.saved_tensors
        E = e2.shape[-1]
        d2 = dinj.reshape(-1, E)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        de = C.gemm_nn(d2, _lp(weight)[:, E:]).view(ctx.eshape) if ctx.needs_input_grad[0] else None
        dw = _half_wgrad(d2, e2, weight, slice(E, 2 * E)) if ctx.needs_input_grad[1] else None
        return de, dw


class _AdapterState(torch.autograd.Function):
    """y = x Ws^T + inj with the addition in the GEMM epilogue."""

    @staticmethod
    def forward(ctx, x, inj, weight):
        C = cuda_backend()
        E = x.shape[-1]
        x2 = x.reshape(-1, E)
        (y,) = sac.run_op("mm", lambda: (C.gemm(x2, _lp(weight)[:, :E], resid=inj.reshape(-1, E),
                                                  out_mode=C.OUT_BF16_RESID),))
        ctx.save_for_backward(x2, weight)
        ctx.xshape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        C = cuda_backend()
        x2, weight = ctx.saved_tensors
        E = x2.shape[-1]
        dy2 = dy.reshape(-1, E)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = C.gemm_nn(dy2, _lp(weight)[:, :E]).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        dinj = dy if ctx.needs_input_grad[1] else None
        dw = _half_wgrad(dy2, x2, weight, slice(0, E)) if ctx.needs_input_grad[2] else None
        return dx, dinj, dw


def adapter_inject(e: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if e.is_cuda:
        return _AdapterInject.apply(e, weight)
    return ref.linear(e, weight[:, e.shape[-1]:])


def adapter_state(x: torch.Tensor, inj: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if x.is_cuda:
        return _AdapterState.apply(x, inj, weight)
    return ref.linear(x, weight[:, :x.shape[-1]]) + inj


def adapter(x: torch.Tensor, e: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    if x.is_cuda:
        return _Adapter.apply(x, e, weight)
    return ref.adapter(x, e, weight)


# ------------------------------------------------------------------------------------------
# norms
# ------------------------------------------------------------------------------------------
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        C = cuda_backend()
        x2 = x.reshape(-1, x.shape[-1])
        y, rstd = C.rmsnorm_fwd(x2, weight, eps)
        ctx.save_for_backward(x2, weight, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        C = cuda_backend()
        x2, weight, rstd = ctx.saved_tensors
        dx, dw = C.rmsnorm_bwd(dy.reshape(x2.shape), x2, weight, rstd, need_dw=ctx.needs_input_grad[1])
        return dx.view(dy.shape), (dw.to(weight.dtype) if dw is not None else None), None


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, x, weight, eps):
        C = cuda_backend()
        a2, x2 = a.reshape(-1, a.shape[-1]), x.reshape(-1, x.shape[-1])
        y, s, rstd = C.add_rmsnorm_fwd(a2, x2, weight, eps)
        ctx.save_for_backward(s, weight, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        C = cuda_backend()
        s, weight, rstd = ctx.saved_tensors
        ds, dw = C.rmsnorm_bwd(dy.reshape(s.shape), s, weight, rstd, need_dw=ctx.needs_input_grad[2])
        ds = ds.view(dy.shape)
        return ds, ds, (dw.to(weight.dtype) if dw is not None else None), None


def rmsnorm(x, weight, eps: float):
    if x.is_cuda:
        return _RMSNorm.apply(x, weight, eps)
    return ref.rmsnorm(x, weight, eps)


def add_rmsnorm(a, x, weight, eps: float):
    if x.is_cuda:
        return _AddRMSNorm.apply(a, x, weight, eps)
    return ref.add_rmsnorm(a, x, weight, eps)


# ------------------------------------------------------------------------------------------
# qk-bias + RoPE, attention, SwiGLU
# ------------------------------------------------------------------------------------------
class _RopeAttention(torch.autograd.Function):
    """qkv [B,S,(H+2Hkv)D] -> causal attention output [B,S,H*D].

    Forward: one pass adds the q/k bias and rotates q,k into a packed copy (the only tensor saved besides the
    output and the row log-sum-exp); the attention kernel reads q, k, v as strided views of that copy.
    Backward: the attention backward writes dq|dk|dv into one packed buffer, which is un-rotated in place and
    handed to the Wqkv GEMMs without a concatenation."""

    @staticmethod
    def forward(ctx, qkv, qk_bias, cos, sin, n_head, n_kv, head_dim, scale):
        C = cuda_backend()
        qkv_r = C.rope_fwd(qkv, qk_bias, cos, sin, n_head, n_kv, head_dim)
        o, lse = sac.run_op("attn", lambda: C.attention_fwd(qkv_r, n_head, n_kv, head_dim, scale))
        ctx.save_for_backward(qkv_r, o, lse, cos, sin)
        ctx.meta = (n_head, n_kv, head_dim, scale, qk_bias is not None)
        return o

    @staticmethod
    def backward(ctx, do):
        C = cuda_backend()
        qkv_r, o, lse, cos, sin = ctx.saved_tensors
        n_head, n_kv, head_dim, scale, has_bias = ctx.meta
        dqkv = C.attention_bwd(do.contiguous(), qkv_r, o, lse, n_head, n_kv, head_dim, scale)
        dqkv, dbias = C.rope_bwd_(dqkv, cos, sin, n_head, n_kv, head_dim, has_bias and ctx.needs_input_grad[1])
        return dqkv, dbias, None, None, None, None, None, None


class _QKVRopeAttention(torch.autograd.Function):
    """x [B,S,E], Wqkv -> causal attention output: the QKV projection adds the q/k bias and rotates q and k in its GEMM
    epilogue (no separate pass over the packed tensor), then the attention kernel runs on the packed rotated tensor.
    Backward: attention backward into one packed buffer, inverse rotation in place, then the two Wqkv GEMMs."""

    @staticmethod
    def forward(ctx, x, weight, qk_bias, cos, sin, n_head, n_kv, head_dim, scale):
        C = cuda_backend()
        B, S, E = x.shape
        x2 = x.reshape(-1, E)
        bias = None if qk_bias is None else qk_bias.detach().float().reshape(-1).contiguous()
        width = (n_head + n_kv) * head_dim
        (qkv_r,) = sac.run_op("mm", lambda: (C.gemm(x2, _lp(weight), out_mode=C.OUT_BF16_ROPE,
                                                    rope=(cos, sin, bias, S, head_dim, width)).view(B, S, -1),))
        o, lse = sac.run_op("attn", lambda: C.attention_fwd(qkv_r, n_head, n_kv, head_dim, scale))
        ctx.save_for_backward(x2, weight, qkv_r, o, lse, cos, sin)
        ctx.meta = (n_head, n_kv, head_dim, scale, qk_bias is not None, x.shape)
        return o

    @staticmethod
    def backward(ctx, do):
        C = cuda_backend()
        x2, weight, qkv_r, o, lse, cos, sin = ctx.saved_tensors
        n_head, n_kv, head_dim, scale, has_bias, xshape = ctx.meta
        dqkv = C.attention_bwd(do.contiguous(), qkv_r, o, lse, n_head, n_kv, head_dim, scale)
        dqkv, dbias = C.rope_bwd_(dqkv, cos, sin, n_head, n_kv, head_dim, has_bias and ctx.needs_input_grad[2])
        d2 = dqkv.view(-1, dqkv.shape[-1])
        dx = C.gemm_nn(d2, _lp(weight)).view(xshape) if ctx.needs_input_grad[0] else None
        dw = _wgrad(d2, x2, weight) if ctx.needs_input_grad[1] else None
        return dx, dw, dbias, None, None, None, None, None, None


def qkv_rope_attention(x, weight, qk_bias, cos, sin, n_head: int, n_kv: int, head_dim: int, scale: float | None = None):
    """Wqkv projection + qk-bias + RoPE + causal attention; the GPU path fuses bias and rotation into the GEMM."""
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    if x.is_cuda and cos.dtype == torch.float32 and cos.shape[0] == x.shape[1] and not _ag_pending(weight):
        return _QKVRopeAttention.apply(x, weight, qk_bias, cos.contiguous(), sin.contiguous(), n_head, n_kv, head_dim,
                                       scale)
    return rope_attention(linear(x, weight), qk_bias, cos, sin, n_head, n_kv, head_dim, scale)


def rope_attention(qkv, qk_bias, cos, sin, n_head: int, n_kv: int, head_dim: int, scale: float | None = None):
    """Fused qk-bias + RoPE + causal attention on a packed qkv tensor; returns [B, S, n_head*head_dim]."""
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    if qkv.is_cuda:
        return _RopeAttention.apply(qkv, qk_bias, cos, sin, n_head, n_kv, head_dim, scale)
    q, k, v = ref.qk_bias_rope(qkv, qk_bias, cos, sin, n_head, n_kv, head_dim)
    o = ref.causal_attention(q, k, v, scale)
    return o.reshape(*qkv.shape[:2], n_head * head_dim)


def qk_bias_rope(qkv, qk_bias, cos, sin, n_head: int, n_kv: int, head_dim: int):
    """Unfused form (used by the inference model, which caches k and v): returns q, k, v as [B,S,H,hd]."""
    if qkv.is_cuda and not torch.is_grad_enabled():
        r = cuda_backend().rope_fwd(qkv, qk_bias, cos, sin, n_head, n_kv, head_dim)
        B, S, _ = r.shape
        wq, wk = n_head * head_dim, n_kv * head_dim
        return (r[..., :wq].view(B, S, n_head, head_dim), r[..., wq:wq + wk].view(B, S, n_kv, head_dim),
                r[..., wq + wk:].view(B, S, n_kv, head_dim))
    return ref.qk_bias_rope(qkv, qk_bias, cos, sin, n_head, n_kv, head_dim)


def causal_attention(q, k, v, scale: float | None = None, q_offset: int = 0):
    """q,k,v: [B,S,H,hd] -> [B,Sq,H,hd] (inference path; keys start at position 0, queries at q_offset)."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if q.is_cuda:
        return cuda_backend().attention_infer(q, k, v, scale, q_offset)
    return ref.causal_attention(q, k, v, scale, q_offset)


def masked_attention(q, k, v, mask, scale: float | None = None):
    """Attention under an explicit boolean mask [B,1,Sq,Sk] (padding / block masks of the eager HF-style model).  The
    fp32 statement on every device: this path serves masked prefill of padded batches, not the training step."""
    if q.is_cuda:
        cuda_backend()._library("attention_masked", "explicit attention mask (eager HF-style model)", strict=False)
    return ref.masked_attention(q, k, v, mask, scale)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h):
        C = cuda_backend()
        ctx.save_for_backward(h)
        return C.swiglu_fwd(h)

    @staticmethod
    def backward(ctx, dy):
        C = cuda_backend()
        (h,) = ctx.saved_tensors
        return C.swiglu_bwd(dy.contiguous(), h)


def swiglu(h):
    if h.is_cuda:
        return _SwiGLU.apply(h)
    return ref.swiglu(h)


# ------------------------------------------------------------------------------------------
# embedding, fused linear + cross-entropy, state init
# ------------------------------------------------------------------------------------------
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, scale):
        C = cuda_backend()
        ctx.save_for_backward(ids, weight)
        ctx.scale = scale
        return C.embedding_fwd(ids, _lp(weight), scale)

    @staticmethod
    def backward(ctx, dy):
        C = cuda_backend()
        ids, weight = ctx.saved_tensors
        if getattr(weight, "_fused_grad", False) and weight.grad is not None:
            if _store_first(weight):
                weight.grad.zero_()          # the scatter-add needs a cleared buffer when nothing was stored before it
            C.embedding_bwd(dy.contiguous(), ids, weight.grad, ctx.scale)
            return None, None, None
        dw = torch.zeros(weight.shape, dtype=torch.float32, device=dy.device)
        C.embedding_bwd(dy.contiguous(), ids, dw, ctx.scale)
        return None, dw.to(weight.dtype), None


def embedding(ids, weight, scale: float = 1.0):
    if weight.is_cuda:
        return _Embedding.apply(ids, weight, scale)
    return ref.embedding(ids, weight, scale)


class _LinearCE(torch.autograd.Function):
    """Loss = mean CE(x W^T * logit_scale) without keeping the logits: the forward walks the rows in
    chunks, keeps (lse, target logit) per row, and already produces dX and dW for a unit loss gradient
    (the scheme of recpre/ops.py:1034-1040); backward only scales them by the incoming gradient."""

    @staticmethod
    def forward(ctx, x, weight, labels, logit_scale, ignore_index, z_reg, telemetry=None):
        C = cuda_backend()
        x2 = x.reshape(-1, x.shape[-1])
        lab = labels.reshape(-1)
        need_grad = x.requires_grad or weight.requires_grad
        loss, dx, dw = C.linear_ce(x2, _lp(weight), lab, logit_scale, ignore_index, z_reg, need_grad=need_grad,
                                   telemetry=telemetry)
        ctx.weight = weight
        if need_grad:
            ctx.save_for_backward(dx, dw)
        ctx.xshape = x.shape
        return loss

    @staticmethod
    def backward(ctx, dloss):
        dx, dw = ctx.saved_tensors
        weight = ctx.weight
        dx = (dx * dloss.to(dx.dtype)).view(ctx.xshape)
        if getattr(weight, "_fused_grad", False) and weight.grad is not None:
            if _store_first(weight):
                torch.mul(dw, dloss.to(dw.dtype), out=weight.grad)
            else:
                weight.grad.addcmul_(dw, dloss.to(dw.dtype))
            return dx, None, None, None, None, None, None
        return dx, (dw * dloss).to(weight.dtype), None, None, None, None, None


def linear_cross_entropy(x, weight, labels, logit_scale: float = 1.0, ignore_index: int = -100, z_reg: float = 0.0,
                         telemetry: torch.Tensor | None = None):
    """Mean cross entropy of ``x W^T * logit_scale`` without materialising the logits.  ``telemetry`` (CUDA path; four
    fp32 zeros) receives the sums over valid rows of the maximal logit, the entropy of the prediction, the L2 norm of
    the logits and lse^2 -- the head statistics the reference's fused head reports (recpre/ops.py:1120-1127)."""
    if x.is_cuda:
        return _LinearCE.apply(x, weight, labels, logit_scale, ignore_index, z_reg, telemetry)
    return ref.linear_cross_entropy(x, weight, labels, logit_scale, ignore_index, z_reg)


def trunc_normal_state(like: torch.Tensor, std: float, seed: int, generator: torch.Generator | None = None):
    """Fresh recurrent state with the shape/dtype/device of ``like``."""
    if like.is_cuda:
        return cuda_backend().trunc_normal(like.shape, std, seed, like.dtype, like.device)
    if generator is None:
        generator = torch.Generator(device="cpu")
        generator.manual_seed(seed)
    return ref.trunc_normal_state(like.shape, std, generator, like.device, like.dtype)
