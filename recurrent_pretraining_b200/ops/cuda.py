"""ctypes binding of the in-tree sm_100a kernel library (``_lib/libb200ops.so``).

Importing this module loads the library and raises if it is missing, so a GPU run can never silently
take a PyTorch fallback.  Every wrapper launches on the current PyTorch CUDA stream and allocates
its outputs through the PyTorch caching allocator; nothing here synchronises the device.

Declared library paths (everything else either runs an in-tree kernel or raises).  Each use is counted in
``LIBRARY_CALLS`` and announced once per process on stderr, so a run that leaves the native kernels shows it:

* ``attention_fwd`` / ``attention_bwd`` with a head dim other than 64, 96 or 128, or with
  ``B200_NATIVE_ATTENTION=0`` / ``B200_NATIVE_ATTENTION_BWD=0`` (comparison switches of the kernel benchmarks):
  torch's scaled-dot-product attention.  ``B200_STRICT_NATIVE=1`` turns these into errors.
* ``attention_infer``: the eager HF model's cached decoding (``models/hf.py``; the serving engine has its own
  flash-decoding kernel and never comes here) always uses torch's attention.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_lib", "libb200ops.so")


def _load() -> C.CDLL:
    if not os.path.exists(_LIB_PATH):
        raise ImportError(
            f"native kernel library not built: {_LIB_PATH}; run `python -m recurrent_pretraining_b200.csrc.build`")
    return C.CDLL(_LIB_PATH)


lib = _load()
_vp, _i, _f, _ll, _ull = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_ulonglong


def _sig(name, argtypes):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = C.c_int
    return fn


_gemm = _sig("b200_gemm", [_vp] * 5 + [_i] * 14 + [_vp, _vp])
_rms_fwd = _sig("b200_rmsnorm_fwd", [_vp] * 6 + [_i, _i, _f, _vp])
_rms_bwd = _sig("b200_rmsnorm_bwd", [_vp] * 7 + [_i, _i, _vp])
_rms_bwd_grid = _sig("b200_rmsnorm_bwd_grid", [_i])
_rope = _sig("b200_rope", [_vp] * 6 + [_i] * 6 + [_vp])
_bias_grad = _sig("b200_bias_grad", [_vp, _vp, _i, _i, _i, _vp])
_swiglu_fwd = _sig("b200_swiglu_fwd", [_vp, _vp, _ll, _i, _vp])
_swiglu_bwd = _sig("b200_swiglu_bwd", [_vp, _vp, _vp, _ll, _i, _vp])
_emb_fwd = _sig("b200_embedding_fwd", [_vp, _vp, _vp, _ll, _i, _f, _ll, _vp, _vp])
_emb_bwd = _sig("b200_embedding_bwd", [_vp, _vp, _vp, _ll, _i, _f, _ll, _vp, _vp])
_trunc_normal = _sig("b200_trunc_normal", [_vp, _ll, _f, _ull, _vp])
_sumsq = _sig("b200_sumsq", [_vp, _ll, _vp, _vp])
_adamw = _sig("b200_adamw", [_vp] * 5 + [_ll, _vp] + [_f] * 9 + [_i, _i, _vp])
_cast = _sig("b200_cast_f32_bf16", [_vp, _vp, _ll, _vp])
_ce_rows = _sig("b200_ce_rows", [_vp] * 6 + [_i] * 4 + [_f, _i, _f, _vp])

_set_2cta = _sig("b200_gemm_set_2cta", [_i])

OUT_BF16, OUT_F32, OUT_F32_ACC, OUT_BF16_RESID, OUT_SWIGLU = range(5)
OUT_BF16_ROPE = 7
OUT_SWIGLU_SAVE = 8     # SwiGLU epilogue that also stores the pre-activation [gate | up] into ``resid``
OUT_DSWIGLU = 9         # input-gradient GEMM whose epilogue applies the gate's derivative (``resid`` = pre-activation)
OUT_BF16_LSE = 10       # head GEMM: bf16 logits + per-tile softmax partials + target logit (fused linear + CE)
_set_lse = _sig("b200_gemm_set_lse", [_vp, _vp, _vp, _f])
_ce_finish = _sig("b200_ce_finish", [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _f, _i, _f, _i, _vp])
_set_rope = _sig("b200_gemm_set_rope", [_vp, _vp, _vp, _i, _i, _i])


def set_gemm_2cta(enable: bool) -> bool:
    """Select the 2-CTA (cta_group::2, 256-row tiles) GEMM where it applies; returns the previous setting."""
    return bool(_set_2cta(int(enable)))

_set_raster = _sig("b200_gemm_set_raster", [_i])


def set_gemm_raster(group: int) -> int:
    """Tile order of the large GEMMs: ``group`` consecutive m tiles are walked across all n tiles before the next
    group (a wave of the persistent grid then covers a near-square block of tiles and re-uses both operand panels from
    L2); 0 = m fastest over the whole matrix.  Returns the previous setting."""
    return int(_set_raster(int(group)))


if os.environ.get("B200_GEMM_RASTER"):
    set_gemm_raster(int(os.environ["B200_GEMM_RASTER"]))

BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launch_count() -> int:
    """Number of native entry-point calls so far (each launches at least one kernel of this library)."""
    return _launches


def _check(rc: int, what: str) -> None:
    global _launches
    _launches += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def _ptr(t):
    return 0 if t is None else t.data_ptr()


# ------------------------------------------------------------------------------------------------
# device status word (bounded waits inside kernels report here instead of hanging)
# ------------------------------------------------------------------------------------------------
_err_words: dict = {}


def err_word(device=None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _err_words.get(dev)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=dev)
        _err_words[dev] = w
    return w


def check_device_status() -> int:
    """Synchronising read of the status word: 0 means no kernel gave up on a wait."""
    code = int(err_word().item())
    if code:
        err_word().zero_()
    return code


# ------------------------------------------------------------------------------------------------
# GEMM family
# ------------------------------------------------------------------------------------------------
def _mat(t: torch.Tensor):
    """(tensor, rows, cols, ld) for a 2-D bf16 matrix whose rows are contiguous."""
    assert t.dim() == 2 and t.dtype == BF16 and t.stride(1) == 1, (t.shape, t.dtype, t.stride())
    return t, t.shape[0], t.shape[1], t.stride(0)


def gemm(a, b, *, a_mn=False, b_mn=False, out=None, out_mode=OUT_BF16, a2=None, resid=None, n_out=None, bn=0,
         max_ctas=0, rope=None, lse=None):
    """C[M,N] (+)= A B^T.  ``a``: [M,K] (or [K,M] if a_mn), ``b``: [N,K] (or [K,N] if b_mn).
    ``rope`` (OUT_BF16_ROPE): (cos [S, D/2] fp32, sin, bias flat fp32 or None, S, D, width of the q+k columns)."""
    a, ar, ac, lda = _mat(a)
    b, br, bc, ldb = _mat(b)
    M, K1 = (ac, ar) if a_mn else (ar, ac)
    N, K = (bc, br) if b_mn else (br, bc)
    K2 = 0
    lda2 = 0
    if a2 is not None:
        a2, a2r, K2, lda2 = _mat(a2)
        assert a2r == M
    assert K == K1 + K2, (K, K1, K2)
    if out_mode in (OUT_SWIGLU, OUT_SWIGLU_SAVE):
        assert N % 2 == 0
        N //= 2
    if n_out is not None:
        N = n_out
    if out is None:
        dt = BF16 if out_mode in (OUT_BF16, OUT_BF16_RESID, OUT_SWIGLU, OUT_BF16_ROPE, OUT_SWIGLU_SAVE, OUT_BF16_LSE) \
            else torch.float32
        if out_mode == OUT_DSWIGLU:      # [dgate | dup]: the tile epilogue writes both halves
            out = torch.empty((M, 2 * N), dtype=BF16, device=a.device)[:, :N]
        else:
            out = torch.empty((M, N), dtype=dt, device=a.device)
    assert out.dim() == 2 and out.stride(1) == 1 and out.shape[0] == M and out.shape[1] == N
    if out_mode in (OUT_SWIGLU_SAVE, OUT_DSWIGLU):
        assert resid is not None and resid.shape == (M, 2 * N) and resid.stride(0) == 2 * N, "pre-activation [M, 2I]"
        if out_mode == OUT_DSWIGLU:
            assert out.stride(0) == 2 * N and out.dtype == BF16, "the output is the first half of an [M, 2I] matrix"
    ld_resid = 0
    if resid is not None:
        assert resid.dtype == BF16 and resid.stride(1) == 1
        ld_resid = resid.stride(0)
    if out_mode == OUT_BF16_ROPE:
        cos, sin, bias, S, D, width = rope
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
        assert cos.shape[-1] * 2 == D and cos.shape[0] >= S and sin.shape == cos.shape, (cos.shape, S, D)
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() >= width)
        _set_rope(_ptr(cos), _ptr(sin), _ptr(bias), int(S), int(D), int(width))
    if out_mode == OUT_BF16_LSE:
        part, tgt, labels, scale = lse     # [M, ceil(N / 256), 4] fp32, [M] fp32, [M] int64, logit scale
        assert part.dtype == torch.float32 and part.is_contiguous() and part.shape == (M, (N + 255) // 256, 4)
        assert tgt.numel() >= M and labels.dtype == torch.int64 and labels.is_contiguous()
        _set_lse(_ptr(part), _ptr(tgt), _ptr(labels), float(scale))
        bn = 256
    rc = _gemm(_ptr(a), _ptr(a2), _ptr(b), _ptr(out), _ptr(resid), M, N, K1, K2, lda, lda2, ldb, out.stride(0),
               ld_resid, int(a_mn), int(b_mn), out_mode, bn, max_ctas, _stream(), _ptr(err_word(a.device)))
    _check(rc, "b200_gemm")
    return out


def gemm_nt(x, w, out=None, accumulate=False, a2=None):
    """x [M,K] @ w[N,K]^T -> bf16 [M,N] (``a2`` continues the K loop against further columns of w)."""
    assert not accumulate
    return gemm(x, w, out=out, a2=a2)


def gemm_nn(dy, w, out=None):
    """dy [M,N] @ w[N,K] -> bf16 [M,K]   (dgrad: B is read MN-major, no transposed weight copy)."""
    return gemm(dy, w, b_mn=True, out=out)


def gemm_tn(dy, x, out=None, accumulate=False, out_dtype=torch.float32):
    """dy[T,N]^T @ x[T,K] -> [N,K]  (wgrad: both operands read MN-major); fp32 out, optional accumulate."""
    if out is None:
        assert not accumulate
        return gemm(dy, x, a_mn=True, b_mn=True, out_mode=OUT_F32 if out_dtype == torch.float32 else OUT_BF16)
    mode = OUT_F32_ACC if accumulate else (OUT_F32 if out.dtype == torch.float32 else OUT_BF16)
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, out_mode=mode)


def split_bf16(x: torch.Tensor):
    """fp32 matrix -> (hi, lo) bf16 with hi + lo = x to ~16 bits of mantissa."""
    hi = x.to(BF16)
    lo = (x - hi.float()).to(BF16)
    return hi, lo


def matmul_f32(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False) -> torch.Tensor:
    """fp32-accurate product of two fp32 matrices on the bf16 tensor cores: each operand is split into a bf16 head and a
    bf16 remainder and ``hi*hi + hi*lo + lo*hi`` is accumulated in fp32 by three tcgen05 GEMMs (the dropped ``lo*lo``
    term is ~2^-16 relative).  Operand conventions as in ``gemm``: C[M,N] = A B^T with ``a`` [M,K] (or [K,M] with
    ``a_mn``) and ``b`` [N,K] (or [K,N] with ``b_mn``).  Used by the preconditioner products of SOAP / Shampoo, which
    would otherwise run as fp32 SIMT GEMMs."""
    assert a.dtype == torch.float32 and b.dtype == torch.float32 and a.dim() == 2 and b.dim() == 2
    ah, al = split_bf16(a.contiguous())
    bh, bl = split_bf16(b.contiguous())
    out = gemm(ah, bh, a_mn=a_mn, b_mn=b_mn, out_mode=OUT_F32)
    gemm(ah, bl, a_mn=a_mn, b_mn=b_mn, out=out, out_mode=OUT_F32_ACC)
    gemm(al, bh, a_mn=a_mn, b_mn=b_mn, out=out, out_mode=OUT_F32_ACC)
    return out


def matmul_f32_supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Shapes the tensor-core path takes: CUDA fp32 matrices whose every extent is a multiple of 8 and at least 128."""
    return (a.is_cuda and b.is_cuda and a.dtype == torch.float32 and b.dtype == torch.float32 and a.dim() == 2
            and b.dim() == 2 and all(d % 8 == 0 and d >= 128 for d in (*a.shape, *b.shape)))


# ------------------------------------------------------------------------------------------------
# norms
# ------------------------------------------------------------------------------------------------
def _w32(w):
    if w is None:
        return None
    return w if w.dtype == torch.float32 else w.float()


def rmsnorm_fwd(x, weight, eps):
    M, E = x.shape
    assert x.dtype == BF16, x.dtype
    x = x.contiguous()
    y = torch.empty_like(x)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    w = _w32(weight)
    _check(_rms_fwd(_ptr(x), 0, _ptr(w), _ptr(y), 0, _ptr(rstd), M, E, eps, _stream()), "rmsnorm_fwd")
    return y, rstd


def add_rmsnorm_fwd(a, x, weight, eps):
    M, E = x.shape
    assert x.dtype == BF16 and a.dtype == BF16 and a.shape == x.shape, (a.dtype, x.dtype, a.shape, x.shape)
    a, x = a.contiguous(), x.contiguous()
    y, s = torch.empty_like(x), torch.empty_like(x)
    rstd = torch.empty(M, dtype=torch.float32, device=x.device)
    w = _w32(weight)
    _check(_rms_fwd(_ptr(x), _ptr(a), _ptr(w), _ptr(y), _ptr(s), _ptr(rstd), M, E, eps, _stream()), "add_rmsnorm_fwd")
    return y, s, rstd


def rmsnorm_bwd(dy, x, weight, rstd, need_dw=True):
    M, E = x.shape
    assert dy.dtype == BF16 and x.dtype == BF16 and x.is_contiguous() and rstd.dtype == torch.float32 \
        and rstd.numel() == M and dy.shape == x.shape, (dy.dtype, x.dtype, rstd.dtype, dy.shape, x.shape)
    dy = dy.contiguous()
    dx = torch.empty_like(x)
    w = _w32(weight)
    need_dw = need_dw and weight is not None
    dw = part = None
    if need_dw:
        dw = torch.empty(E, dtype=torch.float32, device=x.device)
        part = torch.empty((_rms_bwd_grid(M), E), dtype=torch.float32, device=x.device)
    _check(_rms_bwd(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), _ptr(dx), _ptr(part), _ptr(dw), M, E, _stream()),
           "rmsnorm_bwd")
    return dx, dw


# ------------------------------------------------------------------------------------------------
# rope / attention / swiglu
# ------------------------------------------------------------------------------------------------
def _table32(t):
    """The rotary kernels read fp32 tables; a table that followed its module into bf16 is converted (never reinterpreted)."""
    return t if t.dtype == torch.float32 and t.is_contiguous() else t.float().contiguous()


def rope_fwd(qkv, qk_bias, cos, sin, n_head, n_kv, head_dim, pos_ids=None):
    """Packed [B,S,(H+2Hkv)*D] -> packed, q and k biased + rotated, v copied."""
    B, S, W = qkv.shape
    assert qkv.dtype == BF16 and W == (n_head + 2 * n_kv) * head_dim, (qkv.dtype, qkv.shape)
    cos, sin = _table32(cos), _table32(sin)
    assert cos.shape[-1] * 2 == head_dim and (pos_ids is not None or cos.shape[0] >= S), (cos.shape, S, head_dim)
    qkv = qkv.contiguous()
    out = torch.empty_like(qkv)
    bias = None if qk_bias is None else qk_bias.detach().float().contiguous()
    _check(_rope(_ptr(qkv), _ptr(out), _ptr(bias), _ptr(cos), _ptr(sin), _ptr(pos_ids), B * S, S, n_head, n_kv,
                 head_dim, 0, _stream()), "rope_fwd")
    return out


def rope_bwd_(dqkv, cos, sin, n_head, n_kv, head_dim, has_bias, pos_ids=None):
    """In-place inverse rotation of the q/k parts of a packed gradient; returns (dqkv, dbias or None)."""
    B, S, W = dqkv.shape
    assert dqkv.dtype == BF16 and dqkv.is_contiguous() and W == (n_head + 2 * n_kv) * head_dim, (dqkv.dtype, dqkv.shape)
    cos, sin = _table32(cos), _table32(sin)
    assert cos.shape[-1] * 2 == head_dim and (pos_ids is not None or cos.shape[0] >= S), (cos.shape, S, head_dim)
    _check(_rope(_ptr(dqkv), _ptr(dqkv), 0, _ptr(cos), _ptr(sin), _ptr(pos_ids), B * S, S, n_head, n_kv, head_dim, 1,
                 _stream()), "rope_bwd")
    dbias = None
    if has_bias:
        assert n_head == n_kv, "qk_bias with grouped-query attention is not supported"
        width = (n_head + n_kv) * head_dim
        dbias = torch.zeros(width, dtype=torch.float32, device=dqkv.device)
        _check(_bias_grad(_ptr(dqkv), _ptr(dbias), B * S, W, width, _stream()), "bias_grad")
        dbias = dbias.view(2, 1, n_head, head_dim)
    return dqkv, dbias


def linear_swiglu_save(x, w):
    """(silu(x Wg^T) * (x Wu^T), pre-activation [M, 2I]) in one GEMM whose epilogue applies the gate and stores both."""
    M, two_i = x.shape[0], w.shape[0]
    h = torch.empty((M, two_i), dtype=BF16, device=x.device)
    y = gemm(x, w, out_mode=OUT_SWIGLU_SAVE, resid=h)
    return y, h


def dswiglu_dgrad(dy_out, w_proj, h):
    """dh [M, 2I] = dswiglu(dy_out @ w_proj, h): the input-gradient GEMM of the down projection with the derivative of
    the gate in its epilogue (no [M, I] intermediate, no separate elementwise pass)."""
    M, I = dy_out.shape[0], w_proj.shape[1]
    dh = torch.empty((M, 2 * I), dtype=BF16, device=dy_out.device)
    gemm(dy_out, w_proj, b_mn=True, out=dh[:, :I], out_mode=OUT_DSWIGLU, resid=h)
    return dh


def swiglu_fwd(h):
    I = h.shape[-1] // 2
    h = h.contiguous()
    y = torch.empty(*h.shape[:-1], I, dtype=h.dtype, device=h.device)
    _check(_swiglu_fwd(_ptr(h), _ptr(y), h.numel() // (2 * I), I, _stream()), "swiglu_fwd")
    return y


def swiglu_bwd(dy, h):
    I = h.shape[-1] // 2
    dh = torch.empty_like(h)
    _check(_swiglu_bwd(_ptr(dy), _ptr(h), _ptr(dh), h.numel() // (2 * I), I, _stream()), "swiglu_bwd")
    return dh


# ------------------------------------------------------------------------------------------------
# embedding / state init
# ------------------------------------------------------------------------------------------------
def embedding_fwd(ids, w_bf16, scale):
    assert ids.dtype == torch.int64 and w_bf16.dtype == BF16 and w_bf16.is_contiguous(), (ids.dtype, w_bf16.dtype)
    ids = ids.contiguous()
    E = w_bf16.shape[1]
    out = torch.empty(*ids.shape, E, dtype=BF16, device=w_bf16.device)
    _check(_emb_fwd(_ptr(ids), _ptr(w_bf16), _ptr(out), ids.numel(), E, float(scale), w_bf16.shape[0],
                    _ptr(err_word(w_bf16.device)), _stream()), "embedding_fwd")
    return out


def embedding_bwd(dy, ids, grad_f32, scale):
    E = grad_f32.shape[1]
    assert grad_f32.dtype == torch.float32 and grad_f32.is_contiguous()
    assert ids.dtype == torch.int64 and dy.dtype == BF16 and dy.is_contiguous() and dy.numel() == ids.numel() * E
    ids = ids.contiguous()
    _check(_emb_bwd(_ptr(ids), _ptr(dy), _ptr(grad_f32), ids.numel(), E, float(scale), grad_f32.shape[0],
                    _ptr(err_word(grad_f32.device)), _stream()), "embedding_bwd")


def trunc_normal(shape, std, seed, dtype=BF16, device=None):
    if device is None or torch.device(device).type != "cuda":
        device = torch.device("cuda", torch.cuda.current_device())
    out = torch.empty(tuple(shape), dtype=BF16, device=device)
    _check(_trunc_normal(_ptr(out), out.numel(), float(std), int(seed) & 0xFFFFFFFFFFFFFFFF, _stream()), "trunc_normal")
    return out if dtype == BF16 else out.to(dtype)


# ------------------------------------------------------------------------------------------------
# optimizer pieces
# ------------------------------------------------------------------------------------------------
def sumsq_(g_flat, out):
    assert g_flat.dtype == torch.float32 and g_flat.is_contiguous()
    _check(_sumsq(_ptr(g_flat), g_flat.numel(), _ptr(out), _stream()), "sumsq")


def adamw_(p, g, m, v, shadow, gnorm_sq, *, lr, beta1, beta2, eps, wd, step, max_norm=0.0, grad_scale=1.0,
           zero_grad=True, atan2=False):
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    _check(_adamw(_ptr(p), _ptr(g), _ptr(m), _ptr(v), _ptr(shadow), p.numel(), _ptr(gnorm_sq), lr, beta1, beta2, eps,
                  wd, bc1, bc2, max_norm, grad_scale, int(zero_grad), int(atan2), _stream()), "adamw")


def cast_bf16_(src_f32, dst_bf16):
    _check(_cast(_ptr(src_f32), _ptr(dst_bf16), src_f32.numel(), _stream()), "cast")


# ------------------------------------------------------------------------------------------------
# fused linear + cross entropy
# ------------------------------------------------------------------------------------------------
_ce_scratch: dict = {}


def _scratch(key, shape, dtype, device):
    t = _ce_scratch.get(key)
    if t is None or t.shape != torch.Size(shape) or t.device != device:
        t = torch.empty(shape, dtype=dtype, device=device)
        _ce_scratch[key] = t
    return t


def linear_ce(x, w, labels, logit_scale=1.0, ignore_index=-100, z_reg=0.0, need_grad=True, chunk_rows=1024,
              telemetry=None, fused=None):
    """Returns (loss, dx, dw): mean CE over valid labels, and the gradients for a unit loss gradient.

    Rows are processed in chunks.  Fused form (default when the vocabulary is a multiple of 8): the head GEMM's epilogue
    writes bf16 logits and, per (row, 256-column tile), the online-softmax partials and the target's logit; a row kernel
    merges the partials into the log-sum-exp, adds the loss (and, if asked, telemetry: max logit, entropy, logit norm,
    lse^2 summed over valid rows into ``telemetry[0:4]``) and rewrites the bf16 logits in place as the logit gradient;
    then dX chunk = dlogits W and dW += dlogits^T x.  No fp32 logits exist.  ``fused=False`` keeps the older sequence
    (fp32 logits chunk + row kernel), used as a cross-check."""
    T, E = x.shape
    V = w.shape[0]
    dev = x.device
    assert x.dtype == BF16 and w.dtype == BF16 and x.is_contiguous() and w.is_contiguous() and w.shape[1] == E
    assert labels.dtype == torch.int64 and labels.numel() == T, (labels.dtype, labels.shape, T)
    labels = labels.contiguous()
    loss_sum = torch.zeros(1, dtype=torch.float32, device=dev)
    n_valid = (labels != ignore_index).sum().to(torch.float32).reshape(1)
    rows = min(chunk_rows, T)
    if fused is None:
        fused = V % 8 == 0 and os.environ.get("B200_FUSED_CE", "1") == "1"
    dx = torch.empty_like(x) if need_grad else None
    dw = _scratch(("dw", dev), (V, E), torch.float32, dev) if need_grad else None
    if fused:
        tiles = (V + 255) // 256
        logits = _scratch(("logits_bf16", dev), (rows, V), BF16, dev)
        part = _scratch(("lse_part", dev), (rows, tiles, 4), torch.float32, dev)
        tgt = _scratch(("lse_tgt", dev), (rows,), torch.float32, dev)
        for i, r0 in enumerate(range(0, T, rows)):
            r1 = min(T, r0 + rows)
            n = r1 - r0
            lab = labels[r0:r1]
            tgt.zero_()          # rows whose label is ignored (or out of range) keep 0; they do not enter the loss
            gemm(x[r0:r1], w, out=logits[:n], out_mode=OUT_BF16_LSE, lse=(part[:n], tgt, lab, logit_scale))
            _check(_ce_finish(_ptr(part), tiles, _ptr(tgt), _ptr(lab), _ptr(logits), n, V, V, _ptr(loss_sum), 0,
                              _ptr(telemetry), _ptr(n_valid), float(logit_scale), int(ignore_index), float(z_reg),
                              int(need_grad), _stream()), "ce_finish")
            if need_grad:
                gemm(logits[:n], w, b_mn=True, out=dx[r0:r1])
                gemm(logits[:n], x[r0:r1], a_mn=True, b_mn=True, out=dw, out_mode=OUT_F32 if i == 0 else OUT_F32_ACC)
    else:
        logits = _scratch(("logits", dev), (rows, V), torch.float32, dev)
        dlog = _scratch(("dlogits", dev), (rows, V), BF16, dev) if need_grad else None
        for i, r0 in enumerate(range(0, T, rows)):
            r1 = min(T, r0 + rows)
            n = r1 - r0
            gemm(x[r0:r1], w, out=logits[:n], out_mode=OUT_F32)
            _check(_ce_rows(_ptr(logits), _ptr(labels[r0:r1]), _ptr(dlog), _ptr(loss_sum), 0, _ptr(n_valid), n, V, V, V,
                            float(logit_scale), int(ignore_index), float(z_reg), _stream()), "ce_rows")
            if need_grad:
                gemm(dlog[:n], w, b_mn=True, out=dx[r0:r1])
                gemm(dlog[:n], x[r0:r1], a_mn=True, b_mn=True, out=dw, out_mode=OUT_F32 if i == 0 else OUT_F32_ACC)
    loss = (loss_sum / n_valid.clamp(min=1.0)).reshape(())
    return loss, dx, dw


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------
def _views(qkv_r, n_head, n_kv, D):
    B, S, _ = qkv_r.shape
    wq, wk = n_head * D, n_kv * D
    q = qkv_r[..., :wq].view(B, S, n_head, D)
    k = qkv_r[..., wq:wq + wk].view(B, S, n_kv, D)
    v = qkv_r[..., wq + wk:].view(B, S, n_kv, D)
    return q, k, v


LIBRARY_CALLS: dict = {}


def _library(op: str, why: str, strict: bool = True) -> None:
    """Account for a call that leaves the in-tree kernels."""
    if strict and os.environ.get("B200_STRICT_NATIVE", "0") == "1":
        raise RuntimeError(f"{op}: {why}, and B200_STRICT_NATIVE=1 forbids the library path")
    if op not in LIBRARY_CALLS:
        import sys

        print(f"[b200] {op}: library path ({why})", file=sys.stderr, flush=True)
    LIBRARY_CALLS[op] = LIBRARY_CALLS.get(op, 0) + 1


def _sdpa(q, k, v, scale, causal=True):
    import torch.nn.functional as F

    H, Hk = q.shape[2], k.shape[2]
    return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal,
                                          scale=scale, enable_gqa=H != Hk).transpose(1, 2)


def attention_fwd(qkv_r, n_head, n_kv, D, scale):
    """Causal attention over a packed, already rotated qkv tensor -> (o [B,S,H*D], lse [B,H,S] or None)."""
    B, S, _ = qkv_r.shape
    from . import attention as A

    if A.native_supported(D, S):
        return A.fwd(qkv_r, n_head, n_kv, D, scale)
    _library("attention_fwd", f"head dim {D} has no native kernel" if A.ENABLED else "B200_NATIVE_ATTENTION=0")
    q, k, v = _views(qkv_r, n_head, n_kv, D)
    o = _sdpa(q, k, v, scale)
    return o.reshape(B, S, n_head * D), torch.empty(0, device=qkv_r.device)


def _attention_bwd_library(do, qkv_r, n_head, n_kv, D, scale):
    """Backward through the library attention (recomputes its forward); used for head dims the native kernels do
    not cover."""
    B, S, W = qkv_r.shape
    _library("attention_bwd", f"head dim {D} has no native kernel or the native backward is switched off")
    with torch.enable_grad():
        leaf = qkv_r.detach().requires_grad_(True)
        q, k, v = _views(leaf, n_head, n_kv, D)
        out = _sdpa(q, k, v, scale).reshape(B, S, n_head * D)
        (dqkv,) = torch.autograd.grad(out, leaf, do)
    return dqkv.contiguous()


def attention_bwd(do, qkv_r, o, lse, n_head, n_kv, D, scale):
    """Gradient w.r.t. the packed rotated qkv tensor, returned packed as [B,S,(H+2Hkv)*D]."""
    from . import attention as A

    if lse.numel():
        return A.bwd(do, qkv_r, o, lse, n_head, n_kv, D, scale)
    return _attention_bwd_library(do, qkv_r, n_head, n_kv, D, scale)


def attention_infer(q, k, v, scale, q_offset=0):
    """Inference attention: q [B,Sq,H,D] against cached k,v [B,Sk,Hk,D]; query i sits at position q_offset+i."""
    Sq, Sk = q.shape[1], k.shape[1]
    _library("attention_infer", "eager HF model with a KV cache", strict=False)
    # the library attention is only ever given densely packed operands (a strided batch view of a static cache
    # made its kernel fault)
    if k.shape[0] > 1 and k.stride(0) != k.shape[1] * k.stride(1):
        k, v = k.contiguous(), v.contiguous()
    if Sq == Sk and q_offset == 0:
        return _sdpa(q, k, v, scale, causal=True)
    if Sq == 1:
        return _sdpa(q, k, v, scale, causal=False)
    import torch.nn.functional as F

    qi = torch.arange(Sq, device=q.device)[:, None] + q_offset
    ki = torch.arange(Sk, device=q.device)[None, :]
    mask = ki <= qi
    H, Hk = q.shape[2], k.shape[2]
    return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                          scale=scale, enable_gqa=H != Hk).transpose(1, 2)
