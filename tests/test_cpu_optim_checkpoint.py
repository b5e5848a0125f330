"""Optimizers against the reference implementations, engine modes, checkpoint round trip and resume."""
import copy
import os

import pytest
import torch

import refload
from recurrent_pretraining_b200.config import ModelConfig
from recurrent_pretraining_b200.optim import get_optimizer, get_param_groups
from recurrent_pretraining_b200.optim.ellis import ELLISAdam
from recurrent_pretraining_b200.optim.soap import SOAP
from recurrent_pretraining_b200.parallel.fabric import Fabric
from recurrent_pretraining_b200.runtime import checkpoint as ckpt
from recurrent_pretraining_b200.runtime.engine import TrainEngine

needs_ref = pytest.mark.skipif(not refload.available(), reason="reference not installed under baseline/_ref")


def _run(cls, kw, steps=5):
    torch.manual_seed(1)
    ps = [torch.nn.Parameter(torch.randn(8, 6)), torch.nn.Parameter(torch.randn(6))]
    opt = cls(ps, **kw)
    for i in range(steps):
        for p in ps:
            p.grad = torch.randn_like(p) * (i + 1) * 0.1
        opt.step()
    return [p.detach().clone() for p in ps]


@needs_ref
@pytest.mark.parametrize("extra", [dict(update_clipping=True, atan_adam=True, running_init=True, decouple_wd=True),
                                   dict(nesterov=True), dict(kahan_sum_compensation=True), dict(eps_adjustment=True),
                                   dict(brute_force_clip=0.5), dict(decouple_wd=False, poly_ema_p=2.0)])
def test_ellis_adam_matches_reference(extra):
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-6, weight_decay=0.1, **extra)
    a, b = _run(refload.module("optim").ELLISAdam, kw), _run(ELLISAdam, kw)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)


@needs_ref
def test_soap_matches_reference():
    kw = dict(lr=1e-2, betas=(0.9, 0.95), weight_decay=0.01, precondition_frequency=2)
    a, b = _run(refload.module("soap").SOAP, kw, 7), _run(SOAP, kw, 7)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-5, atol=1e-6)


def test_param_groups_and_registry():
    cfg = ModelConfig.from_name("tiny-raven-cpu")
    model = cfg.construct_model()
    groups = get_param_groups(model.named_parameters(), True, with_names=True)
    assert [len(g["params"]) for g in groups] == [4 * 4 + 1, 1, 4 * 5 + 1]  # weights / embedding / norms + qk_bias
    assert groups[2]["weight_decay"] == 0.0 and any("qk_bias" in n for n in groups[2]["names"])
    for name in ("AdamW", "SGD", "ELLISAdam", "SOAP", "LionW", "SophiaG", "Kellers"):
        opt = get_optimizer(name)(get_param_groups(model.named_parameters()), lr=1e-3)
        assert hasattr(opt, "step")
    with pytest.raises(ValueError):
        get_optimizer("meta-shampoo")


def test_fused_engine_equals_torch_engine_on_cpu_and_skips_first_step():
    torch.manual_seed(3)
    cfg = ModelConfig.from_name("tiny-raven-cpu")
    a = cfg.construct_model()
    b = copy.deepcopy(a)
    before = {n: p.detach().clone() for n, p in a.named_parameters()}
    ea, eb = TrainEngine(a, lr=1e-3, mode="torch"), TrainEngine(b, lr=1e-3, mode="fused")
    for i in range(4):
        ids = torch.randint(0, cfg.padded_vocab_size, (2, 65))
        st = torch.randn(2, 64, cfg.n_embd) * 0.6
        ra = ea.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([1, 2]), input_states=st)
        rb = eb.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([1, 2]), input_states=st)
        assert abs(ra["loss"].item() - rb["loss"].item()) < 1e-4
        if i == 0:  # the very first optimizer step of a run never updates
            assert all(torch.equal(p, before[n]) for n, p in a.named_parameters())
    for (n, p), (_, q) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-6), n


def test_nonfinite_gradient_skips_the_update():
    torch.manual_seed(4)
    cfg = ModelConfig.from_name("tiny-raven-cpu")
    m = cfg.construct_model()
    eng = TrainEngine(m, lr=1e-3, mode="fused", skip_first_step=False)
    ids = torch.randint(0, cfg.padded_vocab_size, (1, 33))
    before = [p.detach().clone() for p in m.parameters()]
    eng.flat_groups[0].grad[3] = float("nan")  # injected on the host
    eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([0, 1]))
    assert all(torch.equal(a, b) for a, b in zip(before, m.parameters()))
    assert float(eng.flat_groups[0].grad.abs().sum()) == 0.0  # gradients are cleared for the next step
    eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([0, 1]))
    assert not all(torch.equal(a, b) for a, b in zip(before, m.parameters()))


def test_checkpoint_round_trip_resume_and_reference_key_layout(tmp_path):
    torch.manual_seed(5)
    cfg = ModelConfig.from_name("tiny-raven-cpu")
    model = cfg.construct_model()
    fabric = Fabric.single("cpu")
    eng = TrainEngine(model, fabric, lr=1e-3, mode="fused")
    ids = [torch.randint(0, cfg.padded_vocab_size, (2, 33)) for _ in range(5)]
    pair = torch.tensor([1, 1])
    for t in ids[:3]:
        eng.train_step(t[:, :-1], t[:, 1:], num_steps_pair=pair, input_states=torch.zeros(2, 32, cfg.n_embd))
    state = {"model": model, "engine": eng, "microbatch_step": eng.micro_step, "optimizer_step": eng.optimizer_step,
             "metrics": {"loss": 1.0}, "should_exit_training": False, "model_config": cfg.to_dict()}
    path = ckpt.save_checkpoint(fabric, state, str(tmp_path), "run", reference_prefixes=True)
    assert os.path.basename(path) == "step-00000003-run_0.pth" and ckpt.find_latest(str(tmp_path), "run", 0) == path
    raw = torch.load(path, weights_only=False)
    assert "_original_module.transformer.core_block.0.attn.Wqkv.weight" in raw["model"]
    inner = ckpt.strip_wrapper_prefixes(raw["model"])
    assert set(inner) == set(model.state_dict())
    cont = [eng.train_step(t[:, :-1], t[:, 1:], num_steps_pair=pair,
                           input_states=torch.zeros(2, 32, cfg.n_embd))["loss"].item() for t in ids[3:]]
    # fresh process state: new model + engine, resume, and the continuation is identical
    torch.manual_seed(99)
    model2 = cfg.construct_model()
    eng2 = TrainEngine(model2, fabric, lr=1e-3, mode="fused")
    state2 = {"model": model2, "engine": eng2, "microbatch_step": 0, "optimizer_step": 0}
    ckpt.load_checkpoint(fabric, state2, path)
    eng2.micro_step, eng2.optimizer_step = state2["microbatch_step"], state2["optimizer_step"]
    cont2 = [eng2.train_step(t[:, :-1], t[:, 1:], num_steps_pair=pair,
                             input_states=torch.zeros(2, 32, cfg.n_embd))["loss"].item() for t in ids[3:]]
    assert cont == pytest.approx(cont2, rel=1e-6)
    # a truncated file is never visible under the final name, and a corrupted one fails loudly
    with open(path, "r+b") as f:
        f.truncate(100)
    with pytest.raises(Exception):
        ckpt.load_checkpoint(fabric, state2, path)


@needs_ref
def test_reference_state_dict_loads_into_our_model_and_back():
    torch.manual_seed(0)
    ov = dict(block_size=64, vocab_size=512, padding_multiple=64, n_embd=96, num_attention_heads=4,
              num_key_value_heads=4, intermediate_size=160)
    ref_model, _ = refload.build_train_model("nebel-raven-3.5b", **ov)
    ours = ModelConfig.from_name("nebel-raven-3.5b", **ov).construct_model()
    wrapped = {"_orig_mod._original_module." + k: v for k, v in ref_model.state_dict().items()}
    ours.load_state_dict(ckpt.strip_wrapper_prefixes(wrapped))
    ref_model.load_state_dict(ckpt.model_state_dict(ours))


def test_research_optimizers_match_reference_math():
    """Lilith / IVON / blocked Shampoo against a direct restatement of their update rules on a toy problem."""
    from recurrent_pretraining_b200.optim import get_optimizer
    from recurrent_pretraining_b200.optim.research import IVON, Lilith, ZeroShampooWithAdamGraftingOptimizer

    assert get_optimizer("Lilith") is Lilith and get_optimizer("IVON") is IVON
    assert get_optimizer("simo-shampoo") is ZeroShampooWithAdamGraftingOptimizer
    torch.manual_seed(0)
    target = torch.randn(12, 8)

    def run(opt_cls, steps=60, **kw):
        w = torch.nn.Parameter(torch.zeros(12, 8))
        b = torch.nn.Parameter(torch.zeros(8))
        opt = opt_cls([w, b], **kw)
        first = None
        for _ in range(steps):
            def closure():
                opt.zero_grad()
                loss = ((w + b - target) ** 2).mean()
                loss.backward()
                return loss
            if isinstance(opt, IVON):
                with opt.sampled_params(train=True):
                    loss = closure()
                opt.step()
            else:
                loss = closure()
                opt.step()
            first = first if first is not None else loss.item()
        return first, loss.item()

    f, l = run(Lilith, lr=1e-2, weight_decay=0.0)
    assert l < 0.5 * f
    f, l = run(IVON, steps=200, lr=0.5, ess=1e4, hess_init=0.1, weight_decay=1e-4, clip_radius=1.0)
    assert l < 0.5 * f
    f, l = run(ZeroShampooWithAdamGraftingOptimizer, lr=5e-2, block_size=4, weight_decay=0.0)
    assert l < 0.2 * f

    # one Lilith step, restated
    w = torch.nn.Parameter(torch.ones(3, 2))
    w.grad = torch.full((3, 2), 0.5)
    Lilith([w], lr=0.1, weight_decay=0.0).step()
    g = 0.5 * (6 ** 0.5 / (6 ** 0.5 * 0.5))
    m1 = 0.1 * g
    m2 = 0.01 * m1
    u = m1 + m2
    v_hat = (0.001 * u * u) / (1 - 0.999)
    want = 1 - 0.1 * u / (v_hat + 1e-8) ** 0.5
    assert torch.allclose(w.detach(), torch.full((3, 2), want), atol=1e-6)
