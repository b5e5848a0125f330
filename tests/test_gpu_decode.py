"""Decode-side kernels and the native decode engine against the PyTorch statements / the eager HF model."""
import math

import pytest
import torch

from recurrent_pretraining_b200.config import ModelConfig
from recurrent_pretraining_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


@pytest.fixture(scope="module")
def small_model():
    from recurrent_pretraining_b200.models.hf import RavenForCausalLM

    torch.manual_seed(0)
    cfg = ModelConfig.from_name("smoke-raven-96", mean_recurrence=4)
    return RavenForCausalLM.from_training_model(cfg.construct_model()).to(torch.bfloat16).cuda().eval()


@pytest.mark.parametrize("B,N,K", [(1, 480, 480), (8, 1440, 480), (33, 2560, 1280), (64, 4096, 5280), (5, 200, 136),
                                   (1, 5280, 5280), (8, 5280, 17920), (16, 15840, 5280), (8, 20000, 512)])
def test_skinny_gemm_matches_matmul(small_model, B, N, K):
    from recurrent_pretraining_b200.engine.decode import DecodeEngine

    eng = DecodeEngine(small_model, max_batch=2, max_len=64, use_graphs=False)
    x, w = _bf(B, K), _bf(N, K, scale=0.05)
    eng.work = torch.zeros(64 * 8192, device="cuda")
    y = eng._linear(x, w)
    want = x.float() @ w.float().T
    assert (y.float() - want).abs().max().item() < 0.02 * math.sqrt(K) * 0.05 * 4 + 0.02 * want.abs().max().item()
    assert not eng.work.any(), "the stream-K accumulator must be handed back cleared"


def test_swiglu_from_accumulator():
    from recurrent_pretraining_b200.engine import decode as D
    from recurrent_pretraining_b200.ops import cuda as K

    T, I = 3, 1000
    acc = torch.randn(T, 2 * I, device="cuda") * 2
    h = acc.bfloat16()
    y = torch.empty(T, I, dtype=torch.bfloat16, device="cuda")
    K._check(D._swiglu_acc(acc.data_ptr(), y.data_ptr(), T, I, K._stream()), "swiglu_acc")
    assert torch.equal(y, K.swiglu_fwd(h)) and not acc.any()


@pytest.mark.parametrize("E", [5280, 2048, 96, 100])
@pytest.mark.parametrize("a_kind", ["f32", "bf16", "none"])
def test_add_rmsnorm_pair(E, a_kind):
    from recurrent_pretraining_b200.engine import decode as D
    from recurrent_pretraining_b200.ops import cuda as K

    torch.manual_seed(E)
    rows, eps = 3, 1e-6
    x = _bf(rows, E)
    a = {"f32": torch.randn(rows, E, device="cuda"), "bf16": _bf(rows, E), "none": None}[a_kind]
    w1, w2 = torch.rand(E, device="cuda") + 0.5, torch.rand(E, device="cuda") + 0.5
    y1, y2 = torch.empty_like(x), torch.empty_like(x)
    s = (x.float() + (a.float() if a is not None else 0)).bfloat16().float()

    def norm(t, w):
        return ((t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)).bfloat16().float() * w).bfloat16().float()

    want1 = norm(s, w1)
    want2 = norm(want1, w2)
    a_in = a.clone() if a is not None else None
    K._check(D._norm_pair(K._ptr(a_in), int(a_kind == "f32"), x.data_ptr(), w1.data_ptr(), w2.data_ptr(), y1.data_ptr(),
                          y2.data_ptr(), rows, E, eps, K._stream()), "add_rmsnorm_pair")
    assert torch.allclose(y1.float(), want1, atol=3e-2, rtol=2e-2)
    assert torch.allclose(y2.float(), want2, atol=3e-2, rtol=2e-2)
    if a_kind == "f32":
        assert not a_in.any(), "the fp32 accumulator is cleared after reading"
    y1b = torch.empty_like(x)
    a_in = a.clone() if a is not None else None
    K._check(D._norm_pair(K._ptr(a_in), int(a_kind == "f32"), x.data_ptr(), w1.data_ptr(), 0, y1b.data_ptr(), 0, rows, E,
                          eps, K._stream()), "add_rmsnorm_pair")
    assert torch.equal(y1b, y1)


def test_rope_append_and_decode_attention():
    from recurrent_pretraining_b200.engine import decode as D
    from recurrent_pretraining_b200.ops import cuda as K

    B, H, Dh, Lmax = 3, 5, 96, 80
    lens = torch.tensor([17, 80, 41], dtype=torch.int32, device="cuda")
    pos = (lens - 1).to(torch.int32)
    kc, vc = _bf(B, Lmax, H, Dh), _bf(B, Lmax, H, Dh)
    qkv = _bf(B, 3 * H * Dh)
    bias = torch.randn(2, 1, H, Dh, device="cuda") * 0.1
    cos, sin = (t.cuda() for t in ref.rope_tables(Dh, Lmax))
    q = torch.empty(B, H * Dh, dtype=torch.bfloat16, device="cuda")
    # fp32 input (the stream-K accumulator, cleared by the kernel) must give the same result as the bf16 input
    acc = qkv.float()
    q32, kc32, vc32 = torch.empty_like(q), kc.clone(), vc.clone()
    K._check(D._rope_append(acc.data_ptr(), bias.contiguous().data_ptr(), cos.data_ptr(), sin.data_ptr(),
                            pos.data_ptr(), q32.data_ptr(), kc32.data_ptr(), vc32.data_ptr(), B, H, H, Dh, Lmax,
                            K._stream(), 1), "rope_append")
    K._check(D._rope_append(qkv.data_ptr(), bias.contiguous().data_ptr(), cos.data_ptr(), sin.data_ptr(),
                            pos.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, H, H, Dh, Lmax, K._stream(), 0),
             "rope_append")
    assert torch.equal(q32, q) and torch.equal(kc32, kc) and torch.equal(vc32, vc) and not acc.any()
    for b in range(B):
        p = int(pos[b])
        qr, kr, vr = ref.qk_bias_rope(qkv[b:b + 1, None], bias, cos[p:p + 1], sin[p:p + 1], H, H, Dh)
        assert torch.allclose(q[b].float(), qr.reshape(-1).float(), atol=2e-2)
        assert torch.allclose(kc[b, p].float(), kr[0, 0].float(), atol=2e-2)
        assert torch.equal(vc[b, p], vr[0, 0])
    splits = 4
    part_o = torch.empty(B * H * splits * Dh, device="cuda")
    part_ml = torch.empty(B * H * splits * 2, device="cuda")
    out = torch.empty_like(q)
    K._check(D._decode_attn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), out.data_ptr(),
                            part_o.data_ptr(), part_ml.data_ptr(), B, H, H, Dh, Lmax, splits, Dh ** -0.5, K._stream()),
             "decode_attention")
    for b in range(B):
        L = int(lens[b])
        want = ref.causal_attention(q[b].view(1, 1, H, Dh).float(), kc[b:b + 1, :L].float(), vc[b:b + 1, :L].float(),
                                    None, L - 1)
        assert torch.allclose(out[b].float(), want.reshape(-1), atol=2e-2, rtol=2e-2), b


def test_kl_exit_kernel_matches_torch():
    from recurrent_pretraining_b200.engine import decode as D
    from recurrent_pretraining_b200.ops import cuda as K

    B, V = 4, 4096
    prev = torch.log_softmax(torch.randn(B, V, device="cuda"), -1)
    logits = torch.randn(B, V, device="cuda") * 2
    logits[1] = prev[1] + 3.0  # same distribution as before -> KL 0 -> exits
    want = torch.nn.functional.kl_div(torch.log_softmax(logits, -1), prev, reduction="none", log_target=True).sum(-1)
    prev_buf = prev.clone()
    kl = torch.zeros(B, device="cuda")
    exited = torch.zeros(B, dtype=torch.int32, device="cuda")
    steps = torch.zeros(B, dtype=torch.int32, device="cuda")
    tok = torch.zeros(B, dtype=torch.int64, device="cuda")
    live = torch.full((1,), B, dtype=torch.int32, device="cuda")
    K._check(D._kl_exit(logits.data_ptr(), prev_buf.data_ptr(), kl.data_ptr(), exited.data_ptr(), steps.data_ptr(),
                        tok.data_ptr(), live.data_ptr(), B, V, 5e-4, 6, 1, K._stream()), "kl_exit")
    assert torch.allclose(kl, want, rtol=1e-3, atol=1e-5)
    assert exited.tolist() == [0, 1, 0, 0] and int(live) == B - 1
    assert torch.equal(tok, logits.argmax(-1)) and steps.tolist() == [7, 7, 7, 7]
    assert torch.allclose(prev_buf, torch.log_softmax(logits, -1), atol=1e-4)


@pytest.mark.parametrize("use_graphs", [False, True])
def test_engine_matches_eager_model(small_model, use_graphs):
    from recurrent_pretraining_b200.engine.decode import DecodeEngine

    torch.manual_seed(1)
    B, P, new = 2, 24, 6
    ids = torch.randint(0, 4000, (B, P), device="cuda")
    eng = DecodeEngine(small_model, max_batch=B, max_len=64, num_steps=4, use_graphs=use_graphs)
    toks, stats = eng.generate(ids, new, init_scale=0.0)
    assert stats["device_status"] == 0 and toks.shape == (B, P + new)
    # the eager model, teacher-forced with the engine's tokens, must predict (nearly) the same next tokens
    out = small_model(toks[:, :-1], num_steps=4, init_scale=0.0)
    pred = out.logits[:, P - 1:, :]
    top2 = pred.topk(2, dim=-1)
    chosen = torch.gather(pred, -1, toks[:, P:].unsqueeze(-1)).squeeze(-1)
    assert bool((chosen >= top2.values[..., 0] - 0.15).all()), (chosen, top2.values[..., 0])


def test_engine_with_programmatic_dependent_launch(small_model, monkeypatch):
    """The captured token graph with programmatic launch edges (each kernel triggers its successor at entry and waits
    for its predecessor before it reads; the skinny GEMM requests weight tiles before that wait) decodes correctly."""
    from recurrent_pretraining_b200.engine import decode as D

    torch.manual_seed(1)
    B, P, new = 2, 24, 6
    ids = torch.randint(0, 4000, (B, P), device="cuda")
    monkeypatch.setattr(D, "PDL", True)
    toks, stats = D.DecodeEngine(small_model, max_batch=B, max_len=64, num_steps=4).generate(ids, new, init_scale=0.0)
    assert stats["device_status"] == 0 and toks.shape == (B, P + new)
    pred = small_model(toks[:, :-1], num_steps=4, init_scale=0.0).logits[:, P - 1:, :]
    chosen = torch.gather(pred, -1, toks[:, P:].unsqueeze(-1)).squeeze(-1)
    assert bool((chosen >= pred.max(-1).values - 0.15).all())


def test_engine_kl_exit_and_latent_reuse(small_model):
    from recurrent_pretraining_b200.engine.decode import DecodeEngine

    torch.manual_seed(2)
    B, P = 2, 16
    ids = torch.randint(0, 4000, (B, P), device="cuda")
    eng = DecodeEngine(small_model, max_batch=B, max_len=48, num_steps=4, max_steps=8)
    _, never = eng.generate(ids, 4, criterion="kl", exit_threshold=0.0, max_steps=8, init_scale=0.0, check_every=2)
    assert all(s == [8, 8] for s in never["steps"])
    _, always = eng.generate(ids, 4, criterion="kl", exit_threshold=1e9, max_steps=8, init_scale=0.0, check_every=1)
    assert all(s == [1, 1] for s in always["steps"])
    toks, reuse = eng.generate(ids, 4, criterion="kl", exit_threshold=5e-4, max_steps=8, continuous_compute=True)
    assert toks.shape == (B, P + 4) and reuse["device_status"] == 0


def test_engine_kl_exit_matches_eager_adaptive_generation(small_model):
    """Device-side KL exit of the engine against ``generate_with_adaptive_compute`` of the eager model on the same
    weights and a deterministic (all-zero) start state: same per-sequence recurrence counts for every generated token and
    the same tokens.  The threshold is put into the widest gap of the KL values seen along the way, so that bf16
    rounding differences between the two implementations cannot flip a decision."""
    from recurrent_pretraining_b200.engine.decode import DecodeEngine

    torch.manual_seed(3)
    B, P, new, cap = 2, 16, 6, 8
    ids = torch.randint(0, 4000, (B, P), device="cuda")
    common = dict(max_new_tokens=new, criterion="kl", num_steps=cap, init_scale=0.0, do_not_exit_in_prefill=True,
                  return_dict_in_generate=True, do_sample=False)
    probe = small_model.generate(ids, exit_threshold=1e-12, **common)
    vals = sorted(v for tok in probe.scores["exit_values"][1:] for seq in tok for v in seq if v > 0)
    assert len(vals) > 8
    lo, hi = vals[len(vals) // 5], vals[-len(vals) // 5]
    inner = [v for v in vals if lo <= v <= hi]
    gap, thr = max((b / a, (a * b) ** 0.5) for a, b in zip(inner, inner[1:]))
    assert gap > 1.05, "no usable gap between consecutive KL values"
    hf = small_model.generate(ids, exit_threshold=thr, **common)
    hf_steps = [list(s) for s in hf.scores["compute_steps"]]
    eng = DecodeEngine(small_model, max_batch=B, max_len=P + new + 1, num_steps=cap, max_steps=cap)
    toks, stats = eng.generate(ids, new, criterion="kl", exit_threshold=thr, max_steps=cap, init_scale=0.0, check_every=1)
    assert stats["device_status"] == 0
    assert hf_steps[0] == [cap] * B                       # the prompt runs the full depth in both
    assert stats["steps"] == hf_steps[1:], (thr, stats["steps"], hf_steps)
    assert any(s < cap for tok in stats["steps"] for s in tok), "the threshold never fired: the test would be vacuous"
    assert torch.equal(toks, hf.sequences), (toks[:, P:], hf.sequences[:, P:])
