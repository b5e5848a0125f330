"""Evaluation helpers on CPU: checkpoint conversion, lm-eval style scoring, depth comparison, step recording."""
import os

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
