"""Numerics of each sm_100a kernel against the plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

from recurrent_pretraining_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["2cta", "1cta"])
def C(request):
    from recurrent_pretraining_b200.ops import cuda

    old = cuda.set_gemm_2cta(request.param == "2cta")
    yield cuda
    cuda.set_gemm_2cta(old)


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _close(got, want, rtol, atol):
    got, want = got.float(), want.float()
    err = (got - want).abs()
    tol = atol + rtol * want.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g}, worst excess {(err - tol).max().item():.4g}"


GEMM_SHAPES = [(128, 128, 64), (256, 512, 256), (300, 200, 136), (129, 240, 1320), (4096, 480, 528), (64, 96, 72),
               (1024, 1024, 2048), (700, 1304, 264)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nt(C, M, N, K):
    a, b = _rand(M, K), _rand(N, K)
    out = C.gemm_nt(a, b)
    torch.cuda.synchronize()
    assert C.check_device_status() == 0
    _close(out, a.float() @ b.float().T, 2e-2, 2e-2 * math.sqrt(K))


@pytest.mark.parametrize("group", [0, 3, 8, 64])
def test_gemm_tile_raster_orders(C, group):
    """Every raster group size visits every output tile exactly once (partial last group, group > tile rows)."""
    old = C.set_gemm_raster(group)
    try:
        for M, N, K in [(2900, 1304, 136), (1300, 3000, 72)]:     # 12 x 6 and 6 x 12 tiles of 256 x 256
            a, b = _rand(M, K), _rand(N, K)
            _close(C.gemm_nt(a, b), a.float() @ b.float().T, 2e-2, 2e-2 * math.sqrt(K))
            g = torch.ones(N, K, device="cuda")
            dy, x = _rand(M, N), _rand(M, K)
            C.gemm_tn(dy, x, out=g, accumulate=True)              # += : a tile visited twice would show
            _close(g, 1 + dy.float().T @ x.float(), 2e-2, 2e-2 * math.sqrt(M))
    finally:
        C.set_gemm_raster(old)
    assert C.check_device_status() == 0


@pytest.mark.parametrize("bn", [128, 240, 256])
def test_gemm_nt_tile_widths(C, bn):
    a, b = _rand(384, 320), _rand(720, 320)
    out = C.gemm(a, b, bn=bn)
    _close(out, a.float() @ b.float().T, 2e-2, 0.4)
    assert C.check_device_status() == 0


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nn_dgrad(C, M, N, K):
    dy, w = _rand(M, K), _rand(K, N)  # dy [M, K] @ w [K, N]
    out = C.gemm_nn(dy, w)
    _close(out, dy.float() @ w.float(), 2e-2, 2e-2 * math.sqrt(K))
    assert C.check_device_status() == 0


@pytest.mark.parametrize("T,N,K", [(128, 128, 128), (512, 256, 192), (1000, 200, 136), (4096, 480, 528)])
def test_gemm_tn_wgrad_accumulate(C, T, N, K):
    dy, x = _rand(T, N), _rand(T, K)
    want = dy.float().T @ x.float()
    out = C.gemm_tn(dy, x)
    assert out.dtype == torch.float32
    _close(out, want, 1e-2, 1e-2 * math.sqrt(T))
    acc = torch.ones(N, K, device="cuda")
    C.gemm_tn(dy, x, out=acc, accumulate=True)
    _close(acc, want + 1.0, 1e-2, 1e-2 * math.sqrt(T))
    assert C.check_device_status() == 0


def test_gemm_strided_views_and_dual_a(C):
    E, T = 136, 300
    w = _rand(E, 2 * E)
    x, e = _rand(T, E), _rand(T, E)
    y = C.gemm_nt(x, w, a2=e)
    _close(y, torch.cat([x, e], -1).float() @ w.float().T, 2e-2, 0.4)
    dy = _rand(T, E)
    dx = C.gemm_nn(dy, w[:, :E])
    de = C.gemm_nn(dy, w[:, E:])
    _close(dx, dy.float() @ w[:, :E].float(), 2e-2, 0.3)
    _close(de, dy.float() @ w[:, E:].float(), 2e-2, 0.3)
    g = torch.zeros(E, 2 * E, device="cuda")
    C.gemm_tn(dy, x, out=g[:, :E], accumulate=True)
    C.gemm_tn(dy, e, out=g[:, E:], accumulate=True)
    _close(g, dy.float().T @ torch.cat([x, e], -1).float(), 1e-2, 0.3)
    assert C.check_device_status() == 0


def test_gemm_residual_and_swiglu_epilogues(C):
    T, E, I = 260, 136, 256
    x, w, r = _rand(T, E), _rand(E, E), _rand(T, E)
    y = C.gemm(x, w, resid=r, out_mode=C.OUT_BF16_RESID)
    _close(y, x.float() @ w.float().T + r.float(), 2e-2, 0.3)
    fc = _rand(2 * I, E, scale=0.2)
    h = C.gemm(x, fc, out_mode=C.OUT_SWIGLU)
    full = x.float() @ fc.float().T
    want = torch.nn.functional.silu(full[:, :I]) * full[:, I:]
    _close(h, want, 3e-2, 0.05)
    assert C.check_device_status() == 0


@pytest.mark.parametrize("M,E", [(7, 256), (33, 480), (64, 5280), (5, 8200), (1100, 480), (1536, 5280)])
def test_rmsnorm_fwd_bwd(C, M, E):
    x, a = _rand(M, E), _rand(M, E)
    w = torch.rand(E, device="cuda") + 0.5
    y, rstd = C.rmsnorm_fwd(x, w, 1e-6)
    _close(y, ref.rmsnorm(x.float(), w, 1e-6), 1e-2, 1e-2)
    y2, s, rstd2 = C.add_rmsnorm_fwd(a, x, w, 1e-6)
    s_ref = (a.float() + x.float()).bfloat16()
    assert torch.equal(s, s_ref)
    _close(y2, ref.rmsnorm(s_ref.float(), w, 1e-6), 1e-2, 1e-2)
    dy = _rand(M, E)
    dx, dw = C.rmsnorm_bwd(dy, x, w, rstd)
    xr = x.float().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    x32 = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6)
    (x32 * wr).backward(dy.float())
    _close(dx, xr.grad, 2e-2, 2e-2)
    _close(dw, wr.grad, 2e-2, 2e-2 * math.sqrt(M))


def test_rope_fwd_bwd(C):
    B, S, H, D = 2, 64, 5, 96
    qkv = _rand(B, S, 3 * H * D)
    bias = (torch.randn(2, 1, H, D, device="cuda") * 0.1)
    cos, sin = (t.cuda() for t in ref.rope_tables(D, S))
    out = C.rope_fwd(qkv, bias, cos, sin, H, H, D)
    q, k, v = ref.qk_bias_rope(qkv, bias, cos, sin, H, H, D)
    want = torch.cat([q.reshape(B, S, -1), k.reshape(B, S, -1), v.reshape(B, S, -1)], -1)
    _close(out, want, 1e-2, 1e-2)
    # backward of a rotation is the inverse rotation; bias grad is the column sum
    d = _rand(B, S, 3 * H * D)
    dq = d.clone()
    dq, dbias = C.rope_bwd_(dq, cos, sin, H, H, D, True)
    leaf = qkv.float().requires_grad_(True)
    bl = bias.clone().requires_grad_(True)
    q, k, v = ref.qk_bias_rope(leaf, bl, cos, sin, H, H, D)
    torch.cat([q.reshape(B, S, -1), k.reshape(B, S, -1), v.reshape(B, S, -1)], -1).backward(d.float())
    _close(dq, leaf.grad, 2e-2, 2e-2)
    _close(dbias, bl.grad, 2e-2, 0.2)


def test_swiglu_embedding_state(C):
    T, I = 37, 264
    h = _rand(T, 2 * I)
    y = C.swiglu_fwd(h)
    _close(y, ref.swiglu(h.float()), 1e-2, 1e-2)
    dy = _rand(T, I)
    dh = C.swiglu_bwd(dy, h)
    hl = h.float().requires_grad_(True)
    ref.swiglu(hl).backward(dy.float())
    _close(dh, hl.grad, 2e-2, 2e-2)
    V, E = 100, 136
    w = _rand(V, E)
    ids = torch.randint(0, V, (3, 11), device="cuda")
    out = C.embedding_fwd(ids, w, 2.0)
    _close(out, w[ids].float() * 2.0, 1e-2, 1e-3)
    g = torch.zeros(V, E, device="cuda")
    d = _rand(3, 11, E)
    C.embedding_bwd(d, ids, g, 2.0)
    want = torch.zeros(V, E, device="cuda").index_add_(0, ids.reshape(-1), d.reshape(-1, E).float() * 2.0)
    _close(g, want, 1e-3, 1e-3)
    s = C.trunc_normal((1024, 1024), 0.6325, 7).float()
    assert abs(s.mean().item()) < 5e-3 and abs(s.std().item() - 0.6325 * 0.9866) < 1e-2
    assert s.abs().max().item() <= 3 * 0.6325 * 1.01
    s2 = C.trunc_normal((1024, 1024), 0.6325, 8).float()
    assert not torch.equal(s, s2)


def test_adamw_matches_torch(C):
    n = 10007
    p0 = torch.randn(n, device="cuda")
    g0 = torch.randn(n, device="cuda") * 0.01
    p = p0.clone(); g = g0.clone(); m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    shadow = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pt = p0.clone().requires_grad_(True)
    opt = torch.optim.AdamW([pt], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    gn = torch.zeros(1, device="cuda")
    for step in range(1, 4):
        pt.grad = g0.clone() * step
        torch.nn.utils.clip_grad_norm_([pt], 0.5)
        opt.step()
        g.copy_(g0 * step)
        gn.zero_()
        C.sumsq_(g, gn)
        C.adamw_(p, g, m, v, shadow, gn, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=step, max_norm=0.5)
        assert float(g.abs().max()) == 0.0  # gradient zeroed for the next step
    _close(p, pt.detach(), 1e-4, 1e-5)
    _close(shadow, pt.detach(), 1e-2, 1e-3)


def test_linear_ce(C):
    T, E, V = 300, 136, 1000
    x, w = _rand(T, E), _rand(V, E, scale=0.2)
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    loss, dx, dw = C.linear_ce(x, w, labels, chunk_rows=128)
    xl, wl = x.float().requires_grad_(True), w.float().requires_grad_(True)
    want = ref.linear_cross_entropy(xl, wl, labels)
    want.backward()
    assert abs(loss.item() - want.item()) < 2e-3 * max(1.0, abs(want.item()))
    _close(dx, xl.grad, 5e-2, 2e-4)
    _close(dw, wl.grad, 5e-2, 2e-4)


@pytest.mark.parametrize("T,E,V,chunk", [(300, 136, 1000, 128), (700, 264, 4096, 512), (1024, 528, 65536, 1024)])
def test_fused_linear_ce_epilogue_form(C, T, E, V, chunk):
    """Head GEMM with the online-softmax partials in its epilogue + the row kernel that merges them (bf16 logits only):
    loss, z term, both gradients and the telemetry sums against the fp32 statement, and against the older fp32-logits
    sequence."""
    x, w = _rand(T, E), _rand(V, E, scale=0.2)
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    tele = torch.zeros(4, device="cuda")
    loss, dx, dw = C.linear_ce(x, w, labels, logit_scale=0.5, z_reg=1e-3, chunk_rows=chunk, telemetry=tele, fused=True)
    loss, dx, dw = loss.clone(), dx.clone(), dw.clone()
    old_loss, old_dx, old_dw = C.linear_ce(x, w, labels, logit_scale=0.5, z_reg=1e-3, chunk_rows=chunk, fused=False)
    xl, wl = x.float().requires_grad_(True), w.float().requires_grad_(True)
    logits = (xl @ wl.T) * 0.5
    valid = labels != -100
    lse = torch.logsumexp(logits, -1)
    want = torch.nn.functional.cross_entropy(logits, labels, ignore_index=-100) + 1e-3 * (lse[valid] ** 2).mean()
    want.backward()
    assert abs(loss.item() - want.item()) < 2e-3 * max(1.0, abs(want.item()))
    assert abs(loss.item() - old_loss.item()) < 2e-3 * max(1.0, abs(want.item()))
    _close(dx, xl.grad, 5e-2, 3e-2 * float(xl.grad.abs().max()))
    _close(dw, wl.grad, 5e-2, 3e-2 * float(wl.grad.abs().max()))
    _close(dx, old_dx, 5e-2, 3e-2 * float(xl.grad.abs().max()))
    lg = logits.detach()[valid]
    p = torch.softmax(lg, -1)
    ent = -(p * torch.log_softmax(lg, -1)).sum(-1)
    want_t = torch.stack([lg.max(-1).values.sum(), ent.sum(), lg.norm(dim=-1).sum(), (lse.detach()[valid] ** 2).sum()])
    assert torch.allclose(tele, want_t, rtol=2e-2, atol=1e-2 * float(want_t.abs().max())), (tele, want_t)
    assert C.check_device_status() == 0


def _packed_qkv(B, S, H, Hkv, D):
    return _rand(B, S, (H + 2 * Hkv) * D, scale=0.7)


def _attention_reference(qkv, H, Hkv, D, scale):
    B, S, _ = qkv.shape
    wq, wk = H * D, Hkv * D
    q = qkv[..., :wq].reshape(B, S, H, D)
    k = qkv[..., wq:wq + wk].reshape(B, S, Hkv, D)
    v = qkv[..., wq + wk:].reshape(B, S, Hkv, D)
    return ref.causal_attention(q.float(), k.float(), v.float(), scale), (q, k, v)


@pytest.mark.parametrize("B,S,H,Hkv,D", [(2, 256, 5, 5, 96), (1, 200, 3, 3, 64), (1, 512, 2, 2, 128), (1, 384, 4, 2, 96),
                                         (1, 1024, 2, 2, 96), (2, 128, 5, 5, 96), (1, 4096, 3, 3, 96)])
@pytest.mark.parametrize("variant", [1, 2])
def test_flash_attention_forward(C, B, S, H, Hkv, D, variant):
    from recurrent_pretraining_b200.ops import attention as A

    qkv = _packed_qkv(B, S, H, Hkv, D)
    scale = D ** -0.5
    old = A.set_fwd_variant(variant)
    try:
        o, lse = A.fwd(qkv, H, Hkv, D, scale)
    finally:
        A.set_fwd_variant(old)
    torch.cuda.synchronize()
    assert C.check_device_status() == 0
    want, (q, k, v) = _attention_reference(qkv, H, Hkv, D, scale)
    _close(o.view(B, S, H, D), want, 2e-2, 2e-2)
    kk = k.float().repeat_interleave(H // Hkv, dim=2)
    scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), kk) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device="cuda").triu(1)
    want_lse = torch.logsumexp(scores.masked_fill(mask, float("-inf")), dim=-1)
    _close(lse, want_lse, 1e-2, 2e-2)


@pytest.mark.parametrize("B,S,H,Hkv,D", [(2, 256, 5, 5, 96), (1, 200, 3, 3, 64), (1, 512, 2, 2, 128), (1, 384, 4, 2, 96),
                                         (1, 1024, 2, 2, 96), (2, 128, 5, 5, 96), (1, 4096, 3, 3, 96)])
@pytest.mark.parametrize("variant", [1, 2])
def test_flash_attention_backward(C, B, S, H, Hkv, D, variant):
    from recurrent_pretraining_b200.ops import attention as A

    assert A.NATIVE_BWD, "the native attention backward entry point is missing from the built library"
    qkv = _packed_qkv(B, S, H, Hkv, D)
    scale = D ** -0.5
    o, lse = A.fwd(qkv, H, Hkv, D, scale)
    do = (torch.randn(B, S, H * D, device="cuda") * 0.5).bfloat16()
    old = A.set_bwd_variant(variant)
    try:
        dqkv = A.bwd(do, qkv, o, lse, H, Hkv, D, scale)
    finally:
        A.set_bwd_variant(old)
    torch.cuda.synchronize()
    assert C.check_device_status() == 0
    x = qkv.float().requires_grad_(True)
    want, _ = _attention_reference(x, H, Hkv, D, scale)
    want.backward(do.float().view(B, S, H, D))
    wq = H * D
    wk = Hkv * D
    for name, sl in (("dq", slice(0, wq)), ("dk", slice(wq, wq + wk)), ("dv", slice(wq + wk, wq + 2 * wk))):
        got, ref_g = dqkv[..., sl].float(), x.grad[..., sl]
        err = (got - ref_g).abs().max().item()
        assert err <= 3e-2 * ref_g.abs().max().item() + 1e-3, (name, err, ref_g.abs().max().item())


@pytest.mark.parametrize("T,S,H,D,E", [(128, 64, 5, 96, 264), (520, 260, 3, 64, 136), (4096, 4096, 2, 96, 72)])
def test_gemm_rope_epilogue(C, T, S, H, D, E):
    """QKV projection whose epilogue adds the q/k bias and rotates q and k, against GEMM followed by the rope kernel."""
    x, w = _rand(T, E), _rand(3 * H * D, E, scale=0.3)
    bias = torch.randn(2 * H * D, device="cuda") * 0.1
    cos, sin = (t.cuda().contiguous() for t in ref.rope_tables(D, S))
    got = C.gemm(x, w, out_mode=C.OUT_BF16_ROPE, rope=(cos, sin, bias, S, D, 2 * H * D))
    torch.cuda.synchronize()
    assert C.check_device_status() == 0
    qkv = (x.float() @ w.float().T).view(T // S, S, 3 * H * D)
    q, k, v = ref.qk_bias_rope(qkv, bias.view(2, 1, H, D), cos, sin, H, H, D)
    want = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], -1)
    _close(got, want, 2e-2, 2e-2 * math.sqrt(E))


@pytest.mark.parametrize("T,E,I", [(260, 136, 256), (260, 136, 200), (512, 264, 384), (1024, 5280, 1792)])
def test_swiglu_save_and_dswiglu_epilogues(C, T, E, I):
    """Gate-up GEMM that stores the gated product and the pre-activation; down-projection input-gradient GEMM with the
    gate's derivative in its epilogue -- against the fp32 statement of the MLP's forward and backward."""
    x, fc, proj = _rand(T, E), _rand(2 * I, E, scale=0.2), _rand(E, I, scale=0.2)
    y, h = C.linear_swiglu_save(x, fc)
    full = x.float() @ fc.float().T
    _close(h, full, 2e-2, 0.05)
    _close(y, torch.nn.functional.silu(full[:, :I]) * full[:, I:], 3e-2, 0.05)
    dout = _rand(T, E, scale=0.5)
    dh = C.dswiglu_dgrad(dout, proj, h)
    hl = h.float().requires_grad_(True)
    act = torch.nn.functional.silu(hl[:, :I]) * hl[:, I:]
    (act @ proj.float().T).backward(dout.float())
    _close(dh, hl.grad, 3e-2, 0.05 * float(hl.grad.abs().max()))
    assert C.check_device_status() == 0


def test_fused_gated_mlp_matches_unfused_path(C):
    from recurrent_pretraining_b200.ops import functional as ops

    T, E, I = 384, 264, 512
    x = _rand(2, T // 2, E).requires_grad_(True)
    fc = _rand(2 * I, E, scale=0.2).requires_grad_(True)
    proj = _rand(E, I, scale=0.2).requires_grad_(True)
    dout = _rand(2, T // 2, E)
    out = ops.gated_mlp(x, fc, proj)
    out.backward(dout)
    got = (out.detach(), x.grad.clone(), fc.grad.clone(), proj.grad.clone())
    for t in (x, fc, proj):
        t.grad = None
    ref_out = ops.linear(ops.swiglu(ops.linear(x, fc)), proj)
    ref_out.backward(dout)
    for a, b in zip(got, (ref_out.detach(), x.grad, fc.grad, proj.grad)):
        _close(a, b, 3e-2, 0.03 * float(b.float().abs().max()))


FLAGSHIP = [(4096, 5280, 17920, "nt"), (4096, 15840, 5280, "nt"), (2048, 5280, 10560, "nt"),
            (1024, 17920, 5280, "nn"), (5280, 17920, 2048, "tn"), (512, 5280, 65536, "nn")]


@pytest.mark.parametrize("M,N,K,kind", FLAGSHIP)
def test_gemm_flagship_shapes(C, M, N, K, kind):
    """Tile-tail and raster paths of the real model: N = 5280 (22 tiles of 240, 4.76 waves), N = 15840, the K = 17920
    contraction, the dual-A adapter width, a weight gradient and the K = 65536 contraction that keeps the m-fastest
    order.  Compared on a sample of rows against fp32 (the full fp32 product of these shapes would dominate the run)."""
    torch.manual_seed(M + N)
    if kind == "nt":
        a, b = _rand(M, K, scale=0.3), _rand(N, K, scale=0.3)
        out = C.gemm_nt(a, b)
        rows = torch.randint(0, M, (48,), device="cuda")
        want = a[rows].float() @ b.float().T
        got = out[rows]
    elif kind == "nn":
        a, b = _rand(M, K, scale=0.3), _rand(K, N, scale=0.3)
        out = C.gemm_nn(a, b)
        rows = torch.randint(0, M, (48,), device="cuda")
        want = a[rows].float() @ b.float()
        got = out[rows]
    else:   # weight gradient dy^T x into fp32, accumulated twice
        dy, x = _rand(K, M, scale=0.3), _rand(K, N, scale=0.3)
        out = torch.zeros(M, N, device="cuda")
        C.gemm_tn(dy, x, out=out, accumulate=False)
        C.gemm_tn(dy, x, out=out, accumulate=True)
        rows = torch.randint(0, M, (48,), device="cuda")
        want = 2 * (dy[:, rows].float().T @ x.float())
        got = out[rows]
    torch.cuda.synchronize()
    _close(got, want, 2e-2, 0.02 * float(want.abs().max()))
    assert C.check_device_status() == 0


@pytest.mark.parametrize("T,N,K", [(512, 1000, 264), (300, 5280, 520), (4096, 776, 1096)])
def test_gemm_tn_fp32_tiles_through_bulk_stores(C, T, N, K):
    """Weight-gradient GEMM on the pair kernel (M >= 256): fp32 tiles leave through shared memory and bulk tensor stores
    (first contribution) / reductions (accumulation).  Ragged extents in both dimensions, a column-slice output view
    (row pitch larger than the width, as the adapter halves), and values that were there before."""
    dy, x = _rand(T, N), _rand(T, K)
    want = dy.float().T @ x.float()
    tol = 1e-2 * math.sqrt(T)
    full = torch.full((N, 2 * K + 8), 3.0, device="cuda")
    view = full[:, 8:8 + K]
    C.gemm_tn(dy, x, out=view, accumulate=False)
    _close(view, want, 1e-2, tol)
    assert torch.all(full[:, :8] == 3.0) and torch.all(full[:, 8 + K:] == 3.0)     # nothing outside the view
    C.gemm_tn(dy, x, out=view, accumulate=True)
    _close(view, 2 * want, 1e-2, 2 * tol)
    assert torch.all(full[:, :8] == 3.0) and torch.all(full[:, 8 + K:] == 3.0)
    assert C.check_device_status() == 0


def _guarded(rows, cols, pitch, dtype=torch.bfloat16, pad=4096, sentinel=512.0):
    """A [rows, cols] view with row pitch ``pitch`` inside a larger buffer filled with a sentinel value."""
    big = torch.full((pad + rows * pitch + pad,), sentinel, dtype=dtype, device="cuda")
    return big, big[pad:pad + rows * pitch].view(rows, pitch)[:, :cols]


def _guards_intact(big, rows, cols, pitch, pad=4096, sentinel=512.0):
    body = big[pad:pad + rows * pitch].view(rows, pitch)
    return bool((big[:pad] == sentinel).all()) and bool((big[pad + rows * pitch:] == sentinel).all()) and \
        (cols == pitch or bool((body[:, cols:] == sentinel).all()))


def test_bf16_epilogues_write_nothing_outside_their_output(C):
    """Canary check of the staged bf16 epilogues on ragged extents (rows not a multiple of 32, columns not a multiple
    of 64, row pitch wider than the matrix): the bulk stores are clipped by the tensor map, so the sentinel values in
    front of, behind and between the rows of the output must survive -- and the values inside must be right."""
    M, E, I = 260, 136, 200
    x, w = _rand(M, E), _rand(I, E, scale=0.3)
    big, out = _guarded(M, I, I + 8)                                   # plain NT
    C.gemm_nt(x, w, out=out)
    _close(out, x.float() @ w.float().T, 2e-2, 2e-2 * math.sqrt(E))
    assert _guards_intact(big, M, I, I + 8)
    dy = _rand(M, I)
    big, out = _guarded(M, E, E + 24)                                  # NN (input gradient)
    C.gemm_nn(dy, w, out=out)
    _close(out, dy.float() @ w.float(), 2e-2, 2e-2 * math.sqrt(I))
    assert _guards_intact(big, M, E, E + 24)
    fc, proj = _rand(2 * I, E, scale=0.2), _rand(E, I, scale=0.2)      # gated MLP, training forms
    big_y, y = _guarded(M, I, I + 8)
    big_h, h = _guarded(M, 2 * I, 2 * I)
    C.gemm(x, fc, out=y, out_mode=C.OUT_SWIGLU_SAVE, resid=h)
    full = x.float() @ fc.float().T
    _close(h, full, 2e-2, 0.05)
    _close(y, torch.nn.functional.silu(full[:, :I]) * full[:, I:], 3e-2, 0.05)
    assert _guards_intact(big_y, M, I, I + 8) and _guards_intact(big_h, M, 2 * I, 2 * I)
    big_d, dh = _guarded(M, 2 * I, 2 * I)
    dout = _rand(M, E, scale=0.5)
    C.gemm(dout, proj, b_mn=True, out=dh[:, :I], out_mode=C.OUT_DSWIGLU, resid=h)
    hl = h.float().requires_grad_(True)
    (torch.nn.functional.silu(hl[:, :I]) * hl[:, I:] @ proj.float().T).backward(dout.float())
    _close(dh, hl.grad, 3e-2, 0.05 * float(hl.grad.abs().max()))
    assert _guards_intact(big_d, M, 2 * I, 2 * I)
    H, D, S = 2, 96, 130                                               # q/k bias + rotation
    T, W = 2 * S, 3 * H * D
    xq, wq = _rand(T, E), _rand(W, E, scale=0.3)
    bias = torch.randn(2 * H * D, device="cuda") * 0.1
    cos, sin = (t.cuda().contiguous() for t in ref.rope_tables(D, S))
    big, out = _guarded(T, W, W + 16)
    C.gemm(xq, wq, out=out, out_mode=C.OUT_BF16_ROPE, rope=(cos, sin, bias, S, D, 2 * H * D))
    qkv = (xq.float() @ wq.float().T).view(T // S, S, W)
    q, k, v = ref.qk_bias_rope(qkv, bias.view(2, 1, H, D), cos, sin, H, H, D)
    _close(out, torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], -1), 2e-2, 2e-2 * math.sqrt(E))
    assert _guards_intact(big, T, W, W + 16)
    assert C.check_device_status() == 0


def test_atomics_free_kernels_repeat_bit_for_bit(C):
    """Kernels that use no floating-point atomics give the same bits on every run: GEMMs of every layout (each output
    tile has one writer, the k loop runs in one order), the gated-MLP forms, the norm kernels (the weight gradient is a
    two-stage column sum in a fixed order) and the attention forward pass."""
    M, E, I = 1100, 264, 512
    x, w, dy = _rand(M, E), _rand(I, E, scale=0.3), _rand(M, I)
    fc = _rand(2 * I, E, scale=0.2)
    nw = torch.rand(E, device="cuda") + 0.5
    H, D, S = 3, 96, 384
    qkv = _rand(2, S, 3 * H * D, scale=0.5)
    dyn = _rand(M, E)

    def run():
        out = [C.gemm_nt(x, w), C.gemm_nn(dy, w), C.gemm_tn(dy, x)]
        out += list(C.linear_swiglu_save(x, fc))
        y, rstd = C.rmsnorm_fwd(x, nw, 1e-6)
        out += [y, rstd]
        out += list(C.rmsnorm_bwd(dyn, x, nw, rstd))
        o, lse = C.attention_fwd(qkv, H, H, D, 1.0 / math.sqrt(D))
        out += [o, lse]
        torch.cuda.synchronize()
        return [t.clone() for t in out if t is not None]

    first, second = run(), run()
    assert len(first) == len(second) >= 10
    for i, (a, b) in enumerate(zip(first, second)):
        assert torch.equal(a, b), f"output {i} differs between two runs"
    assert C.check_device_status() == 0
