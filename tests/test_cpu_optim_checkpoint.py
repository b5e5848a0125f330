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
    victim = m.transformer.coda[0].attn.proj.weight

    def poison(p):       # injected on the host, after autograd has written the gradient
        p.grad.view(-1)[3] = float("nan")

    handle = victim.register_post_accumulate_grad_hook(poison)
    eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([0, 1]))
    handle.remove()
    assert all(torch.equal(a, b) for a, b in zip(before, m.parameters()))
    eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([0, 1]))   # the next window starts clean
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


def test_trainer_stops_when_a_kernel_wait_timed_out(tmp_path, monkeypatch):
    """A non-zero device status word (a kernel gave up waiting for a peer) must end the run with an error at the next
    point where the loop synchronises; the fault is a fake status on the host, no GPU involved."""
    from recurrent_pretraining_b200.runtime import trainer
    from recurrent_pretraining_b200.settings import parse_cli

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = parse_cli([f"--config={root}/launch_configs/tiny_cpu_gloo.yaml", f"--out_dir={tmp_path}", "--max_steps=6",
                     "--save_step_interval=0", "--save_last_step=false", "--world_batch_size=2", "--block_size=64"])
    calls = {"n": 0}

    def fake_status(self):
        calls["n"] += 1
        return 5 if calls["n"] >= 3 else 0

    monkeypatch.setattr(Fabric, "device_status", fake_status)
    with pytest.raises(RuntimeError, match="bounded wait"):
        trainer.main(cfg)
    assert calls["n"] == 3       # two clean log points, then the error stops the loop


def test_interval_saves_wait_for_the_accumulation_boundary_and_resume_realigns(tmp_path):
    """save_step_interval that is not a multiple of the accumulation steps: the save happens only on a window boundary;
    a forced save inside a window restarts the window at the resume point."""
    from recurrent_pretraining_b200.runtime import trainer

    class Cfg:
        save_step_interval, save_first_step, save_n_min_before_job_done = 3, False, None
        out_dir, run_name = str(tmp_path), "acc"

    torch.manual_seed(0)
    cfg = ModelConfig.from_name("tiny-raven-cpu")
    fabric = Fabric.single("cpu")
    eng = TrainEngine(cfg.construct_model(), fabric, lr=1e-3, mode="fused", grad_accum=2)
    state = {"model": eng.model, "engine": eng, "microbatch_step": 0, "optimizer_step": 0, "is_accumulating": False}
    saved = []
    for step in range(1, 7):
        ids = torch.randint(0, cfg.padded_vocab_size, (1, 33))
        eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([0, 1]))
        state.update(microbatch_step=eng.micro_step, is_accumulating=eng.is_accumulating())
        before = set(os.listdir(tmp_path / "checkpoints-sane-ddp")) if (tmp_path / "checkpoints-sane-ddp").exists() else set()
        trainer.maybe_save(Cfg, fabric, state)
        after = set(os.listdir(tmp_path / "checkpoints-sane-ddp")) if (tmp_path / "checkpoints-sane-ddp").exists() else set()
        if after - before:
            saved.append(step)
    assert saved == [6]          # step 3 is inside a window (3 % 2 != 0): skipped; step 6 is due and on a boundary
    # forced save inside a window, then resume: the next window starts at the resume point
    ids = torch.randint(0, cfg.padded_vocab_size, (1, 33))
    eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([0, 1]))
    state.update(microbatch_step=eng.micro_step, is_accumulating=eng.is_accumulating())
    assert state["is_accumulating"]
    trainer.maybe_save(Cfg, fabric, state, force=True)
    eng2 = TrainEngine(cfg.construct_model(), fabric, lr=1e-3, mode="fused", grad_accum=2)
    state2 = {"model": eng2.model, "engine": eng2, "microbatch_step": 0, "optimizer_step": 0}
    ckpt.load_checkpoint(fabric, state2, ckpt.find_latest(str(tmp_path), "acc", 0))
    assert eng2.micro_step == 7 and eng2.window_base == 7 and not eng2.is_accumulating()
    eng2.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([0, 1]))
    assert eng2.is_accumulating()        # first micro-batch of the realigned window
    out = eng2.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([0, 1]))
    assert out["grad_norm"] is not None and not eng2.is_accumulating()


def test_deferred_update_runs_cover_the_weight_group_once():
    """The part of the update that runs beside the next forward pass: the recurrent core (with the adapter) and the coda
    must be one contiguous run each of the flat weight group, and the runs must tile the buffer without gaps."""
    from recurrent_pretraining_b200.config import ModelConfig
    from recurrent_pretraining_b200.optim.fused import deferred_runs
    from recurrent_pretraining_b200.optim.groups import get_param_groups

    model = ModelConfig.from_name("tiny-raven-cpu").construct_model()
    named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    g = get_param_groups(named, False, with_names=True)[0]
    offsets, off = [], 0
    for p in g["params"]:
        offsets.append(off)
        off += (p.numel() + 127) // 128 * 128
    runs = deferred_runs(g["names"], offsets, [p.numel() for p in g["params"]], off)
    assert [r[0] for r in runs] == [None, "core", "coda"]
    assert runs[0][1] == 0 and runs[-1][2] == off
    assert all(a[2] == b[1] for a, b in zip(runs, runs[1:]))
    for name, o in zip(g["names"], offsets):
        phase = next(r[0] for r in runs if r[1] <= o < r[2])
        want = "core" if (".core_block." in name or ".adapter." in name) else ("coda" if ".coda." in name else None)
        assert phase == want, (name, phase)
    # a layout in which the coda is split by other tensors is refused
    assert deferred_runs(["transformer.coda.0.a", "transformer.prelude.0.a", "transformer.coda.1.a",
                          "transformer.core_block.0.a"], [0, 128, 256, 384], [128] * 4, 512) is None


def _run_three(cls, kw, steps=6, sampled=False):
    """A matrix, a vector and a 'vocabulary-sized' matrix under a fixed stream of gradients."""
    torch.manual_seed(1)
    ps = [torch.nn.Parameter(torch.randn(12, 8)), torch.nn.Parameter(torch.randn(6)),
          torch.nn.Parameter(torch.randn(32, 8))]
    opt = cls(ps, **kw)
    targets = [torch.randn_like(p) for p in ps]
    for i in range(steps):
        if sampled:                                   # variational optimizers draw the weights they evaluate
            torch.manual_seed(100 + i)
            with opt.sampled_params(train=True):
                for p in ps:
                    p.grad = None
                sum(((p - t) ** 2).sum() for p, t in zip(ps, targets)).backward()
        else:
            for p in ps:
                p.grad = torch.randn_like(p) * (i + 1) * 0.1
            if i % 2 == 0 and hasattr(opt, "update_hessian"):
                opt.update_hessian()                  # Sophia: the Hessian estimate is refreshed every k steps
        opt.step()
    return [p.detach().clone() for p in ps]


@needs_ref
@pytest.mark.parametrize("name,kw,sampled", [
    ("SophiaG", dict(lr=1e-2, betas=(0.9, 0.95), rho=0.05, weight_decay=0.1), False),
    ("SophiaG", dict(lr=1e-2, betas=(0.9, 0.95), rho=1e-4, weight_decay=0.0, maximize=True), False),
    ("Lilith", dict(lr=1e-2), False),
    ("IVON", dict(lr=1e-2, ess=100.0), True),
    ("ZeroShampooWithAdamGraftingOptimizer", dict(lr=1e-2, block_size=4, start_preconditioning=2), False),
    ("OrthogonalNesterov", dict(lr=1e-2, vocab_dim=32, weight_decay=0.1), False),
])
def test_other_optimizers_match_reference_classes(name, kw, sampled):
    """Step-for-step against the reference's own optimizer classes (recpre/optim.py), same constructor keywords.
    The reference's OrthogonalNesterov never accumulates the moments of its AdamW branch; ``frozen_moments`` selects
    that arithmetic for the comparison (the default here accumulates them)."""
    from recurrent_pretraining_b200.optim import others, research

    mine = getattr(others, name, None) or getattr(research, name)
    with torch.compiler.set_stance("force_eager"):                 # the reference decorates helpers with torch.compile
        want = _run_three(getattr(refload.module("optim"), name), kw, sampled=sampled)
    got = _run_three(mine, dict(kw, frozen_moments=True) if name == "OrthogonalNesterov" else kw, sampled=sampled)
    for a, b in zip(got, want):
        assert torch.allclose(a, b, rtol=1e-5, atol=2e-6), float((a - b).abs().max())


def test_orthogonal_nesterov_trains_the_adam_branch_by_default():
    from recurrent_pretraining_b200.optim.others import OrthogonalNesterov

    torch.manual_seed(0)
    w, e, b = (torch.nn.Parameter(torch.randn(8, 16)), torch.nn.Parameter(torch.randn(32, 16)),
               torch.nn.Parameter(torch.randn(16)))
    before = [p.detach().clone() for p in (w, e, b)]
    opt = OrthogonalNesterov([w, e, b], lr=0.1, vocab_dim=32, weight_decay=0.0, zeropower_iters=5)
    for p in (w, e, b):
        p.grad = torch.randn_like(p)
    opt.step()
    # matrix branch: the step has norm 0.1 * lr * sqrt(numel); Adam branch: first step moves every entry by ~lr
    assert abs(float((w - before[0]).norm()) - 0.1 * 0.1 * (w.numel() ** 0.5)) < 1e-4
    assert abs(float((e - before[1]).abs().mean()) - 0.1) < 1e-3 and abs(float((b - before[2]).abs().mean()) - 0.1) < 1e-3
    assert "momentum_buffer" in opt.state[w] and "exp_avg_sq" in opt.state[e]


def test_lion_update_matches_its_definition_and_reports_update_alignment():
    from recurrent_pretraining_b200.optim.others import LionW

    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(5, 7))
    opt = LionW([p], lr=1e-2, betas=(0.9, 0.99), weight_decay=0.1, fused=True)      # unknown keywords are tolerated
    assert opt.param_groups[0]["initial_lr"] == 1e-2 and opt.get_post_step_metrics() == {}
    w, m = p.detach().clone(), torch.zeros(5, 7)
    for _ in range(3):
        g = torch.randn(5, 7)
        p.grad = g.clone()
        opt.step()
        u = 0.9 * m + 0.1 * g
        w = w * (1 - 1e-2 * 0.1) - 1e-2 * torch.sign(u)
        m = 0.99 * m + 0.01 * g
        assert torch.allclose(p.detach(), w, atol=1e-6)
    cos = opt.get_post_step_metrics()["update_cos_sim"]
    assert abs(float(cos) - float((u * u.sign()).sum() / (u.norm() * u.sign().norm()))) < 1e-5


def test_trainer_logs_the_reference_metric_names(tmp_path):
    """One short CPU run through ``trainer.main``: the JSONL log carries this framework's keys and the reference's names
    for the same quantities (train.py:566-636), per-source mixture state included when there are two sources."""
    import json

    from recurrent_pretraining_b200.runtime import trainer
    from recurrent_pretraining_b200.settings import parse_cli

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = parse_cli([f"--config={root}/launch_configs/tiny_cpu_gloo.yaml", f"--out_dir={tmp_path}", "--max_steps=4",
                     "--save_step_interval=0", "--save_last_step=false", "--world_batch_size=2", "--block_size=64",
                     "--log_step_interval=2", "--run_name=names"])
    trainer.main(cfg)
    rows = [json.loads(line) for line in open(tmp_path / "logs" / "names.jsonl")]
    last = rows[-1]
    for key in ("local_loss", "local_ppl", "microbatch_step", "optimizer_step", "steps/second", "seconds/step",
                "tokens/second", "remaining_time", "total_tokens", "total_time", "global_loss", "global_train_ppl",
                "global_grad_norm", "total_FLOPs", "FLOP/S", "model_flop_utilization", "lr"):
        assert key in last, key
    assert last["microbatch_step"] == 4 and last["remaining_time"] == 0 and last["tokens/second"] > 0
    assert abs(last["steps/second"] * last["seconds/step"] - 1) < 1e-9 and last["total_FLOPs"] > 0
