"""Evaluation helpers on CPU: checkpoint conversion, lm-eval style scoring, depth comparison, step recording."""
import os

import pytest
import torch

from recurrent_pretraining_b200.config import ModelConfig

TINY = dict(block_size=64, vocab_size=256, padding_multiple=64, n_embd=64, num_attention_heads=4, num_key_value_heads=4,
            intermediate_size=96, n_layers_in_recurrent_block=2, n_layers_in_prelude=1, n_layers_in_coda=1,
            mean_recurrence=3, mean_backprop_depth=2)


class ByteTok:
    eos_token_id = 0

    def encode(self, s, add_special_tokens=False):
        return [b % 255 + 1 for b in s.encode()]

    def decode(self, toks):
        return bytes((t - 1) % 256 for t in toks).decode("latin1")


def _checkpoint(tmp_path):
    torch.manual_seed(0)
    cfg = ModelConfig.from_name("nebel-raven-3.5b", **TINY)
    model = cfg.construct_model()
    path = os.path.join(tmp_path, "step-00000008-run_0.pth")
    sd = {"_orig_mod._original_module." + k: v for k, v in model.state_dict().items()}  # the reference's wrapper prefix
    torch.save({"model": sd, "model_config": cfg, "microbatch_step": 8}, path)
    return cfg, model, path


def test_checkpoint_converts_to_hf_folder_with_parity(tmp_path):
    from recurrent_pretraining_b200.evaluate.convert_to_hf import convert
    from recurrent_pretraining_b200.models.hf import RavenForCausalLM

    cfg, model, path = _checkpoint(str(tmp_path))
    out = os.path.join(tmp_path, "hf")
    rep = convert(path, out, dtype=torch.float32)
    assert rep["max_logit_diff_vs_training_model"] < 1e-4
    assert rep["cache_consistent"], rep
    assert os.path.exists(os.path.join(out, "config.json")) and os.path.exists(os.path.join(out, "conversion_report.json"))
    again = RavenForCausalLM.from_pretrained(out)
    a = dict(model.named_parameters())["transformer.core_block.0.attn.Wqkv.weight"]
    b = dict(again.named_parameters())["transformer.core_block.0.attn.Wqkv.weight"]
    assert torch.allclose(a, b)
    # the reference's entry point: output folder named like the checkpoint, tokenizer files copied beside the weights
    from recurrent_pretraining_b200.evaluate.convert_to_hf import hf_implementation_test_and_upload

    tok_dir = os.path.join(tmp_path, "tok")
    os.makedirs(tok_dir)
    open(os.path.join(tok_dir, "tokenizer.json"), "w").write("{}")
    rep2 = hf_implementation_test_and_upload(path, tok_dir, device="cpu", out_dir=os.path.join(tmp_path, "eval"),
                                             upload=False, compare_to_pretrain_implementation=True)
    target = os.path.join(tmp_path, "eval", "step-00000008-run_0")
    assert rep2["cache_consistent"] and os.path.exists(os.path.join(target, "config.json"))
    assert os.path.exists(os.path.join(target, "tokenizer.json"))


def test_lm_eval_style_scoring(tmp_path):
    from recurrent_pretraining_b200.evaluate.lm_eval_wrapper import RecurrentLM

    cfg, model, path = _checkpoint(str(tmp_path))
    lm = RecurrentLM.from_checkpoint(path, ByteTok(), batch_size=2, recurrence=3)
    lm.model.config.state_init = "zero"
    reqs = [("the cat", " sat"), ("a", " b"), ("hello world and more", " text")]
    got = lm.loglikelihood(reqs)
    for (ctx, cont), (ll, greedy) in zip(reqs, got):
        ids = torch.tensor([lm.tok_encode(ctx) + lm.tok_encode(cont)])
        logp = torch.log_softmax(lm._logits(ids[:, :-1]), -1)[0]
        n = len(lm.tok_encode(cont))
        want = logp[-n:].gather(-1, ids[0, -n:, None]).sum().item()
        assert abs(ll - want) < 1e-3 and isinstance(greedy, bool)
    roll = lm.loglikelihood_rolling([("some longer document " * 8,)])
    assert roll[0] < 0
    text = lm.generate_until([("abc", {"until": ["\n"], "max_gen_toks": 5})])
    assert isinstance(text[0], str)


def test_chat_compare_and_step_recorder():
    from recurrent_pretraining_b200.evaluate.chat_compare import compare
    from recurrent_pretraining_b200.evaluate.record_steps import record_steps
    from recurrent_pretraining_b200.models.hf import RavenForCausalLM
    from recurrent_pretraining_b200.models.hf_config import RavenConfig

    torch.manual_seed(0)
    model = RavenForCausalLM(RavenConfig(n_embd=64, n_heads=4, n_layers=4, block_size=64, vocab_size=256,
                                         intermediate_size=96, n_layers_in_recurrent_block=2, n_layers_in_prelude=1,
                                         n_layers_in_coda=1, mean_recurrence=4)).eval()
    tok = ByteTok()
    rows = compare(model, tok.encode, tok.decode, "hi there", recurrences=(1, 4), max_new_tokens=4, adaptive=True)
    assert [r["num_steps"] for r in rows] == [1, 4, 4] and rows[-1]["adaptive"] and rows[-1]["mean_steps"] <= 4
    with record_steps(model, criterion="kl", exit_threshold=1e-2) as rec:
        seq = model.generate(torch.tensor([tok.encode("abc")]), max_new_tokens=5, num_steps=6)
        assert torch.is_tensor(seq)
    s = rec.summary()
    assert s["calls"] == 1 and s["tokens"] >= 5 and 1 <= s["mean_steps"] <= 6
    assert model.generate.__name__ != "patched"
    # one-pass benchmark + step statistics, with a stand-in for the harness (record_steps_in_bench.py:30-78)
    from types import SimpleNamespace

    from recurrent_pretraining_b200.evaluate import record_steps as R

    def harness(wrapper, model_args=None, tasks=None, **kw):
        wrapper.model.generate(torch.tensor([tok.encode("abc")]), max_new_tokens=4, num_steps=6, criterion="kl",
                               exit_threshold=1e-2)
        return {"results": {t: {"acc": 1.0} for t in tasks}}

    results, counts = R.evaluate_with_steps(SimpleNamespace(model=model), ["gsm8k"], model_args="x", simple_evaluate=harness)
    entry = results["results"]["gsm8k"]
    assert entry["adaptive_total_tokens"] == len(counts) >= 4 and 1 <= entry["adaptive_avg_steps"] <= 6
    assert entry["adaptive_min_steps"] <= entry["adaptive_max_steps"] and entry["acc"] == 1.0
    import json
    import tempfile

    path = R.save_step_histogram(counts, os.path.join(tempfile.mkdtemp(), "steps.json"))
    assert sum(json.load(open(path)).values()) == len(counts)
    assert R.parse_gen_kwargs("criterion=kl,exit_threshold=5e-4,continuous_compute=true,num_steps=64") == \
        {"criterion": "kl", "exit_threshold": 5e-4, "continuous_compute": True, "num_steps": 64}
    with pytest.raises(ValueError):
        R.step_statistics([0, 0])


def test_adaptive_compute_wrapper_records_steps(tmp_path):
    from recurrent_pretraining_b200.evaluate.adaptive_eval import AUTO_THRESHOLDS, AdaptiveComputeLM
    from recurrent_pretraining_b200.models.hf import RavenForCausalLM
    from recurrent_pretraining_b200.models.hf_config import RavenConfig

    torch.manual_seed(0)
    cfg = ModelConfig.from_name("nebel-raven-3.5b", **TINY)
    model = RavenForCausalLM(RavenConfig.from_model_config(cfg)).eval()
    lm = AdaptiveComputeLM(model, ByteTok(), criterion="latent-diff", exit_threshold="auto", max_steps=6, max_gen_toks=5,
                           device="cpu")
    assert lm.exit_threshold == AUTO_THRESHOLDS["latent-diff"]
    out = lm.generate_until([("hello", {"until": ["\n"], "max_gen_toks": 5}), ("abc", {"max_gen_toks": 3})])
    assert len(out) == 2 and len(lm.step_log) == 2
    summ = lm.compute_summary()
    assert summ["tokens"] == sum(len(r) for r in lm.step_log) and 1 <= summ["mean_steps"] <= 6
    lm.dump(str(tmp_path / "steps.json"))
    import json

    assert json.load(open(tmp_path / "steps.json"))["criterion"] == "latent-diff"


def test_saturation_eval_and_pass_at_k(tmp_path):
    from recurrent_pretraining_b200.evaluate import pass_at_k as pk
    from recurrent_pretraining_b200.evaluate.local_lm_eval import parse_kv
    from recurrent_pretraining_b200.evaluate.saturation_eval import sample_scores, sweep

    depth = {"d": 0}

    def fake_eval(task):
        d = depth["d"]
        if "gsm8k" in task:
            rows = [{"exact_match": float(i < d), "filter": "flexible-extract"} for i in range(4)] + \
                   [{"exact_match": 1.0, "filter": "strict-match"}]
            return {"samples": {task: rows}}
        return {"samples": {task + "_a": [{"acc": 1.0}], task + "_b": [{"acc": float(d > 2)}]}}

    curve = sweep("gsm8k_cot", [1, 3], lambda d: depth.update(d=d), fake_eval, out_dir=str(tmp_path))
    assert curve == {1: 0.25, 3: 0.75}
    assert torch.load(tmp_path / "saturation_gsm8k_cot_3_0.pth")[3] == [1.0, 1.0, 1.0, 0.0]
    depth["d"] = 4
    assert sample_scores("mmlu", fake_eval("mmlu")) == [1.0, 1.0]
    # unbiased estimator against its definition
    from math import comb

    for n, c, k in ((10, 3, 1), (10, 3, 5), (5, 5, 2), (8, 0, 3), (4, 1, 4)):
        want = 1.0 - (comb(n - c, k) / comb(n, k) if n - c >= k else 0.0)
        assert abs(pk.pass_at_k_estimate(n, c, k) - want) < 1e-12
    docs = [{"prompt": "def add(a, b):\n"}]
    preds = pk.build_predictions([["    return a + b\n", "    return a * b\n"]], docs)
    res = pk.pass_at_k(["assert add(2, 3) == 5"], preds, k=[1, 2], timeout_s=20)
    assert res == {"pass@1": 0.5, "pass@2": 1.0}
    assert pk.build_predictions_instruct([["    return 1\n```\nthanks"]], docs)[0][0].endswith("return 1\n")
    assert parse_kv("pretrained=x/y,mean_recurrence=32,exit_threshold=1e-2,flag=true") == \
        {"pretrained": "x/y", "mean_recurrence": 32, "exit_threshold": 0.01, "flag": True}


def test_adaptive_compute_wrapper_with_a_scripted_depth_schedule():
    """An evaluator object instead of a named criterion: ``NumStepsGenerator`` alternating 2 and 4 recurrences per
    generated token (the reference's eval_alternate_loops example); the recorded steps follow the schedule."""
    from recurrent_pretraining_b200.evaluate.adaptive_eval import AdaptiveComputeLM
    from recurrent_pretraining_b200.models.exit_criteria import NumStepsGenerator
    from recurrent_pretraining_b200.models.hf import RavenForCausalLM
    from recurrent_pretraining_b200.models.hf_config import RavenConfig

    torch.manual_seed(0)
    cfg = ModelConfig.from_name("nebel-raven-3.5b", **TINY)
    model = RavenForCausalLM(RavenConfig.from_model_config(cfg)).eval()
    lm = AdaptiveComputeLM(model, ByteTok(), exit_evaluator=NumStepsGenerator(lambda i: 2 if i % 2 == 0 else 4),
                           max_steps=6, max_gen_toks=4, device="cpu")
    lm.generate_until([("hello", {"max_gen_toks": 4})])
    assert lm.step_log and lm.step_log[0][:4] == [2, 4, 2, 4][:len(lm.step_log[0])], lm.step_log


def test_quick_eval_check_scores_a_training_checkpoint_and_stores_results(tmp_path, monkeypatch):
    """The reference's one-call benchmark of a raw training checkpoint (quick_checkpoint_eval.py:327-390) with a
    stand-in for lm-eval's ``simple_evaluate`` that drives the wrapper's scoring interface."""
    import json

    from recurrent_pretraining_b200.evaluate import lm_eval_wrapper, local_lm_eval

    cfg, model, path = _checkpoint(str(tmp_path))
    calls = {}

    def fake_simple_evaluate(model, tasks, num_fewshot, batch_size, device, limit, random_seed, numpy_random_seed,
                             torch_random_seed):
        calls.update(tasks=tasks, seed=(random_seed, numpy_random_seed, torch_random_seed), fewshot=num_fewshot)
        ll = model.loglikelihood([("the cat", " sat")])
        return {"results": {t: {"acc": 0.5, "ll": ll[0][0]} for t in tasks}, "n": len(tasks)}

    monkeypatch.setattr(lm_eval_wrapper.RecurrentLM, "from_checkpoint",
                        classmethod(lambda cls, p, tok, **kw: cls(model, ByteTok(), **{k: v for k, v in kw.items()})))
    res = local_lm_eval.quick_eval_check(path, "unused-tokenizer-folder", device="cpu", out_dir=str(tmp_path / "eval"),
                                         tasks="arc_easy,piqa", num_fewshot=0, batch_size=2, seed=233, recurrence=3,
                                         simple_evaluate=fake_simple_evaluate)
    assert calls == {"tasks": ["arc_easy", "piqa"], "seed": (233, 233, 233), "fewshot": 0}
    stored = json.loads((tmp_path / "eval" / "results_arc_easy,piqa_step-00000008-run_0_3.json").read_text())
    assert stored["n"] == 2 and stored["results"]["piqa"]["acc"] == 0.5 and res["results"]["arc_easy"]["ll"] < 0
