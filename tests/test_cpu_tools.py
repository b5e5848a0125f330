"""Launch, finetune and serving tools on CPU."""
import os
import sys

import torch
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_slurm_launcher_writes_a_consistent_job(tmp_path):
    import launch_slurm as L

    job = L.parse_and_execute(["--config", "launch_configs/nebel_dp_8xb200.yaml", "--nodes", "4", "--budget_hours", "30",
                               "--timeslot", "720", "--dryrun", "--output_dir", str(tmp_path), "--run_name", "t",
                               "--overwrite_env", "NCCL_DEBUG=INFO FOO=1"])
    text = open(os.path.join(job.log_dir, "t.sbatch")).read()
    assert "#SBATCH --nodes=4" in text and "#SBATCH --gpus-per-node=8" in text and "#SBATCH --time=0-12:00:00" in text
    assert "--nnodes=4 --nproc-per-node=8" in text and "train.py --config=launch_configs/nebel_dp_8xb200.yaml" in text
    assert "export NCCL_DEBUG=INFO" in text and "export FOO=1" in text
    assert L.repetitions_needed(1800, 720) == 3
    cmds = L.submit(job, 3, use_chain=True, dryrun=True)
    assert len(cmds) == 3 and "afterany" in cmds[1]
    assert "salloc --nodes=4" in L.interactive(job)


def test_finetuning_example_learns():
    import finetuning_simple_example as F

    cfg = F.CLISettings(model_name="tiny", dataset_location="synthetic", max_steps=6, batch_size=4, micro_batch_size=2,
                        max_samples=32, max_seq_length=256, optim_config=dict(lr=3e-3, weight_decay=0.0))
    res = F.train(cfg)
    assert res["steps"] == 6 and res["losses"][-1] < 0.7 * res["losses"][0] and res["validations"] == []
    # periodic validation on held-out rows and activation checkpointing, from the command line
    cfg2 = F.parse(["--model_name", "tiny", "--dataset_location", "synthetic", "--max_steps", "4", "--batch_size", "4",
                    "--micro_batch_size", "2", "--max_samples", "40", "--eval_interval", "2", "--compile", "true",
                    "--gradient_checkpointing", "true", "--dataset_config", "main",
                    "--optim_config", '{"lr": 3e-3, "weight_decay": 0.0}'])
    assert cfg2.gradient_checkpointing and cfg2.compile and cfg2.eval_interval == 2
    res2 = F.train(cfg2)
    assert [v["step"] for v in res2["validations"]] == [2, 4]
    assert res2["validations"][-1]["val_loss"] < res2["validations"][0]["val_loss"] and \
        res2["validations"][0]["val_tokens"] > 0
    assert abs(F.wsd_lr(0, 100, 1.0, 0.1, 0.1, 0.001) - 0.1) < 1e-9
    assert F.wsd_lr(50, 100, 1.0, 0.1, 0.1, 0.001) == 1.0 and F.wsd_lr(99, 100, 1.0, 0.1, 0.1, 0.001) < 0.2
    ids, mask = F.tokenize([("a?", "b")], F.ByteTokenizer(), cfg)
    assert mask.sum() == 3 and ids[0, 0] == F.ByteTokenizer.bos  # answer byte + end-of-turn + eos are supervised


def _tiny_hf():
    from recurrent_pretraining_b200.models.hf import RavenForCausalLM
    from recurrent_pretraining_b200.models.hf_config import RavenConfig

    torch.manual_seed(0)
    return RavenForCausalLM(RavenConfig(n_embd=64, n_heads=4, n_layers=4, block_size=64, vocab_size=128,
                                        intermediate_size=96, n_layers_in_recurrent_block=2, n_layers_in_prelude=1,
                                        n_layers_in_coda=1, mean_recurrence=3)).eval()


def test_server_batches_and_matches_direct_generation():
    from recurrent_pretraining_b200.engine import server as S

    model = _tiny_hf()
    sched = S.BatchScheduler(S.ModelBackend(model, max_batch=4), window_ms=50.0, stop_ids=())
    try:
        prompts = [[1, 2, 3, 4], [9, 8, 7, 6], [5, 5, 5]]
        reqs = [sched.submit(p, S.DecodeOptions(max_tokens=5, num_steps=3, init_scale=0.0)) for p in prompts]
        for r in reqs:
            assert r.done.wait(120) and r.error is None, r.error
        # the two 4-token prompts share a batch; the 3-token prompt runs alone
        assert sched.stats["requests"] == 3 and sched.stats["batches"] == 2
        for p, r in zip(prompts, reqs):
            want = model.generate(torch.tensor([p]), max_new_tokens=5, num_steps=3, init_scale=0.0)
            want = (want["sequences"] if isinstance(want, dict) else want)[0, len(p):].tolist()
            assert r.tokens == want
        out = S.handle_completion(sched, {"prompt": [1, 2, 3, 4], "max_tokens": 3, "num_steps": 2})
        assert out["usage"] == {"prompt_tokens": 4, "completion_tokens": 3, "total_tokens": 7}
        assert out["choices"][0]["finish_reason"] == "length"
        app = S.create_app(sched)
        assert {r.path for r in app.routes} >= {"/health", "/v1/models", "/v1/completions"}
        try:
            S.handle_completion(sched, {"prompt": "text without tokenizer"})
            raise AssertionError("expected a ValueError")
        except ValueError:
            pass
    finally:
        sched.close()


def test_example_scripts_run():
    import examples.inference_demo as demo
    import examples.speculative_decoding_demo as spec

    demo.main(["--max_new_tokens", "3"])
    spec.main()
    import examples.trajectory_analysis as traj

    rows = traj.main(["--steps", "6", "--tokens", "3"])
    assert len(rows) == 3 and all(len(r["xy"]) == 7 for r in rows)


def test_nvtx_ranges_mark_the_phases_of_a_step():
    import torch

    from recurrent_pretraining_b200.config import ModelConfig
    from recurrent_pretraining_b200.runtime.engine import TrainEngine
    from recurrent_pretraining_b200.utils import nvtx

    nvtx.enable(True)
    nvtx.reset()
    try:
        cfg = ModelConfig.from_name("tiny-raven-cpu")
        eng = TrainEngine(cfg.construct_model(), lr=1e-3, mode="torch")
        ids = torch.randint(0, cfg.padded_vocab_size, (1, 33))
        eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([1, 1]))
        assert nvtx.opened() == ["forward", "prelude", "recurrence", "coda", "backward"]
    finally:
        nvtx.enable(False)
        nvtx.reset()


def test_rope_formulations_agree():
    import torch

    from recurrent_pretraining_b200.ops import reference as ref
    from recurrent_pretraining_b200.ops import rope_variants as rv

    torch.manual_seed(0)
    B, S, H, D = 2, 17, 3, 8
    x = torch.randn(B, S, H, D)
    cos, sin = ref.rope_tables(D, S, 50000.0)
    want = ref.rope_interleaved(x, cos, sin)
    ang = rv.angles(D, S)
    assert torch.allclose(rv.rope_complex(x, rv.complex_table(D, S)), want, atol=1e-5)
    assert torch.allclose(rv.rope_matrix(x, ang), want, atol=1e-5)
    half = rv.rope_rotate_half(rv.to_half_layout(x), ang)
    assert torch.allclose(rv.from_half_layout(half), want, atol=1e-5)
    assert not torch.allclose(rv.rope_rotate_half(x, ang), want, atol=1e-3)   # the layouts are NOT interchangeable


def test_utils_extras(tmp_path):
    import torch
    import torch.nn.functional as F

    from recurrent_pretraining_b200.utils import extras

    # streaming save / load
    sd = {"a": torch.randn(5, 3), "b": torch.arange(7, dtype=torch.int64), "c": torch.randn(4).bfloat16(),
          "empty": torch.empty(0)}
    with extras.incremental_save(str(tmp_path / "ck.zip")) as sv:
        for k, v in sd.items():
            sv.store(k, v)
        sv.store_meta({"step": 3})
    got, meta = extras.load_incremental(str(tmp_path / "ck.zip"))
    assert meta == {"step": 3} and all(torch.equal(got[k], v) and got[k].dtype == v.dtype for k, v in sd.items())
    assert set(extras.load_incremental(str(tmp_path / "ck.zip"), names=["b"])[0]) == {"b"}
    # chunked CE == plain CE; several ignore ids; vocabulary slice
    torch.manual_seed(0)
    logits, tg = torch.randn(2, 37, 50), torch.randint(0, 50, (2, 37))
    tg[0, :5] = 49
    want = F.cross_entropy(logits.view(-1, 50), torch.where(tg == 49, -100, tg).view(-1), ignore_index=-100)
    assert torch.allclose(extras.chunked_cross_entropy(logits, tg, 16, ignore_indices=[-100, 49]), want, atol=1e-6)
    assert torch.allclose(extras.chunked_cross_entropy(logits, tg, 0, ignore_indices=[-100, 49]), want, atol=1e-6)
    # a restricted vocabulary: the listed ids become classes 0, 1, 2 (recpre/utils.py:489-533)
    few = torch.tensor([[3, 7, 9, -1, 7, 3]])
    lg6 = torch.randn(1, 6, 50)
    sl = extras.chunked_cross_entropy(lg6, few, 4, ignore_indices=[-1], target_range=[3, 7, 9])
    keep = few[0] != -1
    remapped = torch.tensor([0, 1, 2, 1, 0])
    assert torch.allclose(sl, F.cross_entropy(lg6[0][keep][:, [3, 7, 9]], remapped), atol=1e-6)
    loss, kept_logits, kept_targets = extras.chunked_cross_entropy(logits, tg, 16, ignore_indices=[-100, 49],
                                                                   return_logits_targets=True)
    n_kept = int((tg != 49).sum())
    assert torch.allclose(loss, want, atol=1e-6) and kept_logits.shape == (n_kept, 50) and kept_targets.numel() == n_kept
    # exact-match statistics
    V, pad = 11, 10
    labels = torch.tensor([[1, 2, 3, 4, 5, pad], [1, 2, 3, 4, 5, 6]])
    lg = F.one_hot(labels.clamp(max=V - 1), V).float()
    lg[1, 4] = F.one_hot(torch.tensor(0), V).float()        # row 1 misses position 4
    st = extras.batch_exact_match(lg, labels, ["x", "y"], [1, 2], [2, 3], pad)
    assert st[1][2] == [(True, "x"), (True, "y")] and st[2][3] == [(True, "x"), (False, "y")]
    assert st["natural_suffix"][2] == [(True, "x"), (False, "y")]
    red = extras.reduce_memorization_metrics([st], dataset_names=["y"])
    assert red["em/2/3"] == 0.5 and red["em/y/2/3"] == 0.0 and red["em/natural_suffix/unmasked"] == 0.5
    assert extras.flops_per_param(4, 2, 8, 100) == 2 * 100 * 4 + 2 * 4 * 8 * 16
    assert extras.gptneox_tflops(1.0, 1, 1, 8, 2, 16, 32, True) > extras.gptneox_tflops(1.0, 1, 1, 8, 2, 16, 32, False)


def test_optimizer_telemetry_names_and_values():
    """The optimizer-side telemetry (gradient norms per layer, g^2/v RMS, effective Adam learning rates, parameter norms)
    for a torch optimizer and for the flat fused optimizer on the same model and step: same metric names as the
    reference's ``track_gradient_metrics`` and the same numbers from both state layouts."""
    import torch

    from recurrent_pretraining_b200.config import ModelConfig
    from recurrent_pretraining_b200.runtime.engine import TrainEngine
    from recurrent_pretraining_b200.runtime.monitor import adam_effective_lr, optimizer_telemetry

    torch.manual_seed(0)
    cfg = ModelConfig.from_name("tiny-raven-cpu")
    ids = torch.randint(0, cfg.padded_vocab_size, (2, 33))
    pair = torch.tensor([1, 2])
    found = {}
    for mode in ("torch", "fused"):
        torch.manual_seed(1)
        model = cfg.construct_model()
        eng = TrainEngine(model, lr=1e-3, mode=mode, skip_first_step=False)
        for _ in range(2):
            eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=pair)
        if mode == "fused":
            eng._begin_window()            # the flat gradient buffers are not cleared between steps: start a window
        else:
            eng.optimizer.zero_grad(set_to_none=False)
        model(ids[:, :-1], labels=ids[:, 1:], num_steps_pair=pair)["loss"].backward()   # fresh gradients to look at
        found[mode] = optimizer_telemetry(model, eng.optimizer)
    t = found["torch"]
    n_blocks = cfg.n_layers_in_prelude + cfg.n_layers_in_recurrent_block + cfg.n_layers_in_coda
    for i in range(n_blocks):
        for key in (f"query_grad_{i}", f"ffn2_grad_{i}", f"q_effective_lr_{i}", f"k_effective_lr_{i}",
                    f"v_effective_lr_{i}", f"ffn2_effective_lr_{i}"):
            assert key in t, key
    for key in ("avg_RMS", "embed_RMS", "local_l1_grad_norm", "l2_param_norm", "l1_param_norm",
                "core_block_l2_param_norm", "word_embed_l2_param_norm", "model_l2_param_norm"):
        assert key in t and t[key] == t[key], key
    assert t["l2_param_norm"] ** 2 == pytest.approx(t["word_embed_l2_param_norm"] ** 2 + t["model_l2_param_norm"] ** 2,
                                                    rel=1e-5)
    f = found["fused"]
    assert set(f) == set(t)
    for key in ("avg_RMS", "embed_RMS", "l2_param_norm", "query_grad_0", "ffn2_grad_1"):
        assert f[key] == pytest.approx(t[key], rel=2e-3, abs=1e-6), (key, f[key], t[key])
    assert f["ffn2_effective_lr_1"] == f["ffn2_effective_lr_1"]     # a mean of ratios with heavy tails: finite, not compared
    # the effective learning rate of a coordinate whose moments equal its gradient statistics is 1 / |g|
    g = torch.tensor([0.5, -2.0, 1e-12])
    lr = adam_effective_lr(g, g.clone(), g * g, 1e-8)
    assert lr[0].item() == pytest.approx(2.0, rel=1e-4) and lr[1].item() == pytest.approx(0.5, rel=1e-4)


def test_flop_accounting_and_mfu():
    """The analytic FLOP count of the config equals what torch's FLOP counter measures on a meta-device copy of the
    model (the reference's MFU measurement); peak table with the precision multiplier and a B200 entry; MFU triple."""
    from recurrent_pretraining_b200.config import ModelConfig
    from recurrent_pretraining_b200.runtime import monitor as M

    cfg = ModelConfig.from_name("tiny-raven-cpu")
    model = cfg.construct_model()
    total, (n, k) = M.measure_flops(cfg, micro_batch_size=1)
    assert total == pytest.approx(cfg.flops_per_token(cfg.block_size, n, k) * cfg.block_size, rel=1e-6)
    assert M.peak_flops("NVIDIA B200", "bf16-mixed") == 2.25e15
    assert M.peak_flops("NVIDIA B200", "32-true") == 2.25e15 / 2
    assert M.peak_flops("NVIDIA H100 80GB HBM3") == 989e12
    per_token, tflops, mfu = M.mfu_metrics(1000.0, 2, model, "bf16-mixed", True, "NVIDIA B200")
    assert per_token == pytest.approx(total / cfg.block_size)
    assert tflops == pytest.approx(per_token * 1000.0 / 1e12) and mfu == pytest.approx(per_token * 1000.0 / 2 / 2.25e15)
    est = M.estimate_flops_per_token(M.num_params(model), cfg)
    assert est == 3 * (6 * M.num_params(model) + 12 * cfg.n_layer * cfg.num_attention_heads * cfg.head_size * cfg.block_size)


def test_small_helpers(tmp_path, monkeypatch):
    """Rounding / counting / directory conventions / remapping / cycling / closed-form count / abacus groups / loss head."""
    import dataclasses

    import torch.nn as nn

    from recurrent_pretraining_b200.utils import helpers as H

    assert H.find_multiple(65, 64) == 128 and H.find_multiple(128, 64) == 128
    lin = nn.Linear(4, 3)
    lin.bias.requires_grad_(False)
    assert H.num_parameters(lin) == 15 and H.num_parameters(lin, True) == 12 and H.num_parameters(lin, False) == 3
    seq = nn.Sequential(nn.Linear(4, 4), nn.ReLU())
    before = seq[0].weight.clone()
    H.reset_parameters(seq)
    assert not torch.equal(before, seq[0].weight)
    # checkpoint directory conventions
    monkeypatch.chdir(tmp_path)
    (tmp_path / "checkpoints" / "org" / "model").mkdir(parents=True)
    assert H.extend_checkpoint_dir("org/model") == (tmp_path / "checkpoints" / "org" / "model").relative_to(tmp_path)
    with pytest.raises(SystemExit):
        H.check_valid_checkpoint_dir(tmp_path / "checkpoints" / "org" / "model")
    d = tmp_path / "checkpoints" / "org" / "model"
    for name in ("lit_model.pth", "model_config.yaml", "tokenizer.json", "tokenizer_config.json"):
        (d / name).write_text("x")
    H.check_valid_checkpoint_dir(d)
    out = tmp_path / "out"
    out.mkdir()
    H.copy_config_files(d, out)
    assert sorted(p.name for p in out.iterdir()) == ["model_config.yaml", "tokenizer.json", "tokenizer_config.json"]
    assert H.flatten_dict({"a": {"b": 1, "c": {"d": 2}}, "e": 3}) == {"a_b": 1, "a_c_d": 2, "e": 3}

    @dataclasses.dataclass
    class S:
        lr: float = 0.1
        name: str = "x"

    def f(alpha=1, cfg=S(), other=[1, 2]):
        return H.capture_hparams()

    hp = f()
    assert hp["alpha"] == 1 and hp["cfg"] == {"lr": 0.1, "name": "x"} and hp["other"] == "[1, 2]"
    H.save_hyperparameters(S(), out)
    assert "lr: 0.1" in (out / "hyperparameters.yaml").read_text()
    assert H.parse_devices(3) == 3 and H.parse_devices("auto") >= 1
    with pytest.raises(ValueError):
        H.parse_devices(0)
    assert H.get_default_supported_precision(True) in ("bf16-mixed", "16-mixed")
    sd = H.map_old_state_dict_weights({"m.old": 1, "m.keep": 2}, {"old": "new"}, "m.")
    assert sd == {"m.new": 1, "m.keep": 2}
    logits = torch.arange(12.0).view(2, 6)
    lg, tg = H.slice_logits_remap_labels(logits, torch.tensor([5, -1]), [1, 3, 5])
    assert lg.tolist() == [[1.0, 3.0, 5.0], [7.0, 9.0, 11.0]] and tg.tolist() == [2, -1]
    it = H.CycleIterator([1, 2, 3])
    assert [next(it) for _ in range(7)] == [1, 2, 3, 1, 2, 3, 1] and it.epoch == 2
    # closed-form count against a real module stack of the same description
    from recurrent_pretraining_b200.config import ModelConfig

    cfg = ModelConfig.from_name("tiny-raven-cpu")
    est = H.param_count_estimator(cfg.n_embd, 1, cfg.padded_vocab_size, cfg.n_head, cfg.head_size, cfg.n_query_groups,
                                  cfg.intermediate_size)
    E, I, V = cfg.n_embd, cfg.intermediate_size, cfg.padded_vocab_size
    assert est == (3 * E * E + E * E + 3 * E * I + 2 * E) + 2 * V * E + E
    groups = H.get_abacus_param_groups([("abacus.weight", nn.Parameter(torch.zeros(2))), ("w", nn.Parameter(torch.zeros(2))),
                                        ("norm.weight", nn.Parameter(torch.zeros(2)))], 0.1, True, 4.0)
    assert [len(g["params"]) for g in groups] == [1, 1, 1] and groups[1]["weight_decay"] == 0.0
    assert groups[2]["lr"] == pytest.approx(0.4)
    head = H.LinearCrossEntropyLoss(8, 16)
    x, y = torch.randn(5, 8), torch.tensor([1, 2, -100, 4, 15])
    want = torch.nn.functional.cross_entropy(head(x), y, ignore_index=-100)
    assert head(x, y).item() == pytest.approx(want.item(), rel=1e-5)


def test_launcher_snapshot_and_staging(tmp_path):
    """Code snapshot of the working tree and the batch-script lines that stage archives on every node."""
    import tarfile

    import launch_slurm as L

    snap = L.snapshot_working_tree(str(tmp_path), "snap")
    names = tarfile.open(snap).getnames()
    assert "snap/bench.py" in names and "snap/recurrent_pretraining_b200/ops/cuda.py" in names
    assert not any("_lib/" in n or n.startswith("snap/_work") for n in names)          # ignored files stay out
    script = L.stage_archives_script([snap, None])
    assert "sbcast -pf" in script and "tar -xzf" in script and ".unpacked" in script
    with pytest.raises(ValueError):
        L.stage_archives_script(["env.zip"])
    job = L.parse_and_execute(["--config", "launch_configs/nebel_dp_8xb200.yaml", "--nodes", "2", "--snapshot", "--dryrun",
                               "--output_dir", str(tmp_path / "out"), "--run_name", "t"])
    text = job.sbatch_text()
    assert 'cd "$STAGE_DIR/t_code"' in text and "sbcast" in text
    # the reference launcher's remaining options: packed environment, proxy, output sub-folder, partition, its flag names
    job = L.parse_and_execute(["--nodes", "1", "--cast_working_dirs", "--dryrun", "--output_dir", str(tmp_path / "out"),
                               "--run_name", "u", "--environment", "/scratch/envs/torch_env.tar.gz", "--enable_internet",
                               "--proxy", "http://proxy:3128/", "--sub_output_dir_name", "runs_u", "--extended_partition"])
    text = job.sbatch_text()
    assert job.run_from_snapshot == "u_code" and job.log_dir.endswith(os.path.join("out", "runs_u", "slurm"))
    assert "torch_env.tar.gz" in text and 'source "$STAGE_DIR"/torch_env/bin/activate' in text
    assert "export https_proxy=http://proxy:3128/" in text and "#SBATCH --partition=extended" in text
    plain = L.parse_and_execute(["--dryrun", "--output_dir", str(tmp_path / "out"), "--run_name", "v",
                                 "--environment", "/opt/venv"]).sbatch_text()
    assert "source /opt/venv/bin/activate" in plain and "proxy" not in plain


def test_every_listed_reference_symbol_resolves_to_an_object_of_this_package():
    """The reference-name table is the porting index: every target must import, and bare names must be unambiguous."""
    from recurrent_pretraining_b200 import reference_names as ref

    assert len(ref.REFERENCE_NAMES) > 150
    for key in ref.REFERENCE_NAMES:
        obj = ref.resolve(key)
        assert obj is not None, key
        assert ref.where(key).startswith("recurrent_pretraining_b200.")
    from recurrent_pretraining_b200.data.datasets import ParquetStream
    from recurrent_pretraining_b200.optim.soap import SOAP

    assert ref.ParquetStreamPure is ParquetStream and ref.SOAP is SOAP
    with pytest.raises(AttributeError):
        ref.RavenForCausalLM        # two reference files define it (current and legacy): ask by dotted path
    with pytest.raises(KeyError):
        ref.resolve("recpre.nothing.Here")


def test_named_weight_schedules_match_the_mixture_scheduler():
    from recurrent_pretraining_b200.data import scheduler as S

    assert S.GetScheduler(None, 7).get_weight(3) == 7
    assert S.GetScheduler(["step", 8, 10, 0.5], 5).get_weight(25) == 2.0
    assert S.GetScheduler(["linear", 10, 20, 100], 5).get_weight(50) == 15.0
    assert S.GetScheduler(["linear", 10, 20, 100], 5).get_weight(500) == 20.0
    assert abs(S.GetScheduler(["cosine", 10, 0, 100], 0).get_weight(50) - 5.0) < 1e-9
    assert S.GetScheduler([[0, ["const", 3]], [10, ["linear", 3, 9, 10]]], 1).get_weight(15) == 6.0
    assert S.GetScheduler(["base"], 1).get_weight(4) == 0
    assert repr(S.StepWeight(8, 10, 0.5)) == "StepWeight: 8, 10, 0.5"
    with pytest.raises(NotImplementedError):
        S.GetScheduler(["spline", 1], 1)


def test_schedules_take_the_reference_call_forms():
    """``get_lr(step, max_steps, cfg)`` / ``get_batch_size(step, cfg)`` as in the reference's train.py:831-862 beside the
    scalar forms; values from the piecewise definition."""
    import math
    import types

    from recurrent_pretraining_b200.optim.schedules import get_batch_size, get_lr

    cfg = types.SimpleNamespace(optim_config={"lr": 3e-3}, warmup_steps=10, cooldown_steps=20, lr_schedule="cosine",
                                min_lr=1e-4, batch_size_ramp=30, batch_size=50, micro_batch_size=4)
    for step in (0, 5, 10, 40, 80, 81, 95, 100):
        a = get_lr(step, 100, cfg)
        assert a == get_lr(3e-3, step, 10, 100, 20, "cosine", 1e-4)
        if step < 10:
            want = 3e-3 * step / 10
        elif step > 80:
            want = max(3e-3 * (100 - step) / 20, 1e-4)
        else:
            want = 1e-4 + 0.5 * (1 + math.cos(math.pi * (step - 10) / 90)) * (3e-3 - 1e-4)
        assert abs(a - want) < 1e-15, step
    assert get_lr(120, 100, types.SimpleNamespace(**{**vars(cfg), "cooldown_steps": 0})) == 1e-4   # past the end
    cfg.lr_schedule = "linear"
    assert abs(get_lr(55, 100, cfg) - (3e-3 - 0.5 * (3e-3 - 1e-4))) < 1e-15
    assert [get_batch_size(s, cfg) for s in (1, 15, 30, 31, 500)] == [1, math.ceil(0.5 * 12.5), 13, 12, 12]
    assert [get_batch_size(s, 30, 12) for s in (0, 15, 30, 31)] == [1, 6, 12, 12]


def test_fabric_offers_the_hand_written_loop_interface(tmp_path, capsys):
    """A loop written against the reference's fabric (setup / backward / clip_gradients / save / load / log_dict / ...,
    recpre/utils.py:1072-1289) runs on ours: here one process on the CPU with a torch optimizer."""
    from recurrent_pretraining_b200.parallel.fabric import Fabric

    fabric = Fabric.single("cpu")
    fabric.launch()
    assert fabric.seed_everything(7, workers=True) == 7 and fabric.rank == 0 and fabric.local_device.type == "cpu"
    assert fabric.strategy == "SimpleDDP" and fabric.get_prefix_for_checkpoint() == "checkpoints-sane-ddp"
    with fabric.init_module(empty_init=False):
        model = torch.nn.Linear(4, 3)
    model = fabric.setup(model, compile=False)
    opt = fabric.setup_optimizers(torch.optim.SGD(model.parameters(), lr=0.1))
    train, val = fabric.setup_dataloaders([1, 2], [3])
    assert train == [1, 2] and val == [3]
    x = torch.randn(5, 4)
    with fabric.no_backward_sync(model, enabled=True):
        fabric.backward(model(x).pow(2).mean(), model=model)
        assert fabric.no_sync
    assert not fabric.no_sync
    fabric.backward(model(x).pow(2).mean(), model=model)
    norm = fabric.clip_gradients(model, opt, max_norm=1e-3)
    total = torch.sqrt(sum(p.grad.pow(2).sum() for p in model.parameters()))
    assert float(norm) > 1e-3 and abs(float(total) - 1e-3) < 1e-6
    opt.step()
    assert float(fabric.all_reduce(3.0)) == 3.0 and fabric.broadcast({"a": 1}) == {"a": 1}
    fabric.barrier()
    # save / load in the reference layout: <location>_<local rank>.pth, state_dict() of model / optimizer
    state = {"model": model, "optimizer": opt, "microbatch_step": 12, "tokenizer": "kept out on load"}
    fabric.save(str(tmp_path / "ckpt" / "step-00000012-run"), state)
    assert (tmp_path / "ckpt" / "step-00000012-run_0.pth").is_file()
    with pytest.raises(ValueError):
        fabric.save(str(tmp_path / "ckpt" / "step-00000012-run"), state, overwrite=False)
    fresh = torch.nn.Linear(4, 3)
    state2 = {"model": fresh, "optimizer": torch.optim.SGD(fresh.parameters(), lr=0.1), "microbatch_step": 0,
              "tokenizer": "mine"}
    fabric.load(str(tmp_path / "ckpt" / "step-00000012-run"), state2)
    assert torch.equal(fresh.weight, model.weight) and state2["microbatch_step"] == 12 and state2["tokenizer"] == "mine"

    class Sink:
        def __init__(self):
            self.rows = []

        def log_metrics(self, metrics, step=None):
            self.rows.append((metrics, step))

    sink = Sink()
    fabric._loggers = [sink]
    fabric.log_dict({"loss": torch.tensor(1.5), "lr": 0.1}, step=3)
    fabric.log_to_summary({"best": 1.0})
    fabric.log_chart({"ignored": 1})
    assert sink.rows[0] == ({"loss": 1.5, "lr": 0.1}, 3) and sink.rows[1][0] == {"summary/best": 1.0}
    fabric.print("hello", ranks=[0])
    fabric.print("silent", ranks=[1])
    assert capsys.readouterr().out.strip() == "hello"
