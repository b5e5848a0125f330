"""Model-level checks of the CUDA path against the fp32 PyTorch statement of the same model."""
import copy

import pytest
import torch

from recurrent_pretraining_b200.config import ModelConfig
from recurrent_pretraining_b200.runtime.engine import TrainEngine

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("name", ["smoke-raven-96", "tiny-raven-cpu"])
def test_loss_and_grads_match_fp32_reference(name):
    torch.manual_seed(0)
    cfg = ModelConfig.from_name(name)
    cpu_model = cfg.construct_model()
    gpu_model = copy.deepcopy(cpu_model)
    eng = TrainEngine(gpu_model.cuda(), lr=1e-3, skip_first_step=False)
    B, S = 2, 256
    ids = torch.randint(0, cfg.padded_vocab_size, (B, S + 1))
    state = torch.randn(B, S, cfg.n_embd) * 0.6
    pair = torch.tensor([1, 2])
    cpu_model.train()
    out_c = cpu_model(ids[:, :-1], labels=ids[:, 1:], num_steps_pair=pair, input_states=state)
    out_c["loss"].backward()
    gpu_model.train()
    out_g = gpu_model(ids[:, :-1].cuda(), labels=ids[:, 1:].cuda(), num_steps_pair=pair,
                      input_states=state.cuda().bfloat16())
    out_g["loss"].backward()
    torch.cuda.synchronize()
    assert abs(out_g["loss"].item() - out_c["loss"].item()) < 0.03 * abs(out_c["loss"].item())
    ref = dict(cpu_model.named_parameters())
    worst = {}
    for n, p in gpu_model.named_parameters():
        err = _rel(p.grad, ref[n].grad)
        worst[n] = err
    bad = {n: e for n, e in worst.items() if e > 0.08}
    assert not bad, f"gradient mismatch: {sorted(bad.items(), key=lambda kv: -kv[1])[:8]}"
    assert eng.optimizer is not None


def test_repeated_batch_is_memorised():
    torch.manual_seed(1)
    cfg = ModelConfig.from_name("smoke-raven-96")
    with torch.device("cuda"):
        model = cfg.construct_model()
    eng = TrainEngine(model, lr=2e-3, skip_first_step=True)
    ids = torch.randint(0, cfg.padded_vocab_size, (2, 257), device="cuda")
    losses = [eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([1, 2]))["loss"].item()
              for _ in range(8)]
    assert losses[1] == pytest.approx(losses[0], rel=0.02)  # the first optimizer step only clears gradients
    assert losses[-1] < losses[0] - 1.5, losses


def test_sampled_depth_step_runs_and_reports_norm():
    torch.manual_seed(2)
    cfg = ModelConfig.from_name("smoke-raven-96")
    with torch.device("cuda"):
        model = cfg.construct_model()
    eng = TrainEngine(model, lr=1e-3, grad_accum=2)
    ids = torch.randint(0, cfg.padded_vocab_size, (1, 513), device="cuda")
    r1 = eng.train_step(ids[:, :-1], ids[:, 1:])
    assert r1["grad_norm"] is None  # still accumulating
    r2 = eng.train_step(ids[:, :-1], ids[:, 1:])
    assert torch.isfinite(r2["grad_norm"]).all() and r2["grad_norm"].item() > 0


def test_training_dynamics_track_fp32_torch_engine():
    """Six optimizer steps on distinct batches, then the first batch again: the fused bf16 engine must follow the
    fp32 torch.optim.AdamW engine step by step (same clip, same skipped first step, same recurrent state)."""
    torch.manual_seed(3)
    cfg = ModelConfig.from_name("smoke-raven-96")
    cpu_model = cfg.construct_model()
    gpu_model = copy.deepcopy(cpu_model)
    eng_c = TrainEngine(cpu_model, lr=1e-3, mode="torch")
    eng_g = TrainEngine(gpu_model.cuda(), lr=1e-3)
    B, S = 2, 128
    batches = [torch.randint(0, cfg.padded_vocab_size, (B, S + 1)) for _ in range(6)]
    batches.append(batches[0])
    pair = torch.tensor([2, 2])
    lc, lg = [], []
    for i, ids in enumerate(batches):
        state = torch.randn(B, S, cfg.n_embd, generator=torch.Generator().manual_seed(100 + i)) * 0.6
        rc = eng_c.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=pair, input_states=state)
        rg = eng_g.train_step(ids[:, :-1].cuda(), ids[:, 1:].cuda(), num_steps_pair=pair,
                              input_states=state.cuda().bfloat16())
        lc.append(rc["loss"].item())
        lg.append(rg["loss"].item())
        assert abs(rg["grad_norm"].item() - rc["grad_norm"].item()) < 0.1 * rc["grad_norm"].item() + 1e-3, (i, lc, lg)
    for a, b in zip(lc, lg):
        assert abs(a - b) < 0.05 * abs(a) + 0.05, (lc, lg)
    assert lg[-1] < lg[0]  # the re-seen batch is (partly) memorised by both engines
