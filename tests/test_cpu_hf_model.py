"""HF-compatible inference model: parity with the unmodified reference HF file, cache semantics, samplers."""
import pytest
import torch

import refload
from recurrent_pretraining_b200.config import ModelConfig
from recurrent_pretraining_b200.models.exit_criteria import get_adaptive_exit_evaluator
from recurrent_pretraining_b200.models.hf import RavenForCausalLM
from recurrent_pretraining_b200.models.hf_config import RavenConfig
from recurrent_pretraining_b200.models.kv_cache import RecurrentKVCache

needs_ref = pytest.mark.skipif(not refload.available(), reason="reference not installed under baseline/_ref")
SMALL = dict(n_embd=96, n_heads=4, n_layers=8, block_size=128, vocab_size=66048, intermediate_size=160,
             n_layers_in_recurrent_block=4, mean_recurrence=4, n_layers_in_prelude=2, n_layers_in_coda=2)


def _ours(seed=0):
    torch.manual_seed(seed)
    return RavenForCausalLM(RavenConfig(**SMALL)).eval()


def _reference_pair():
    """Reference HF model with our weights.  Only a class attribute is adjusted at run time (transformers 5 wants a
    dict for tied weights); the reference source is untouched."""
    mod = refload.module("raven_modeling_minimal")
    cfgmod = refload.module("raven_config_minimal")
    mod.RavenForCausalLM._tied_weights_keys = {"lm_head.weight": "transformer.wte.weight"}
    ours = _ours()
    theirs = mod.RavenForCausalLM(cfgmod.RavenConfig(**SMALL)).eval()
    theirs.load_state_dict(ours.state_dict())
    return ours, theirs, mod


@needs_ref
def test_forward_logits_loss_and_cached_decoding_match_reference():
    ours, theirs, mod = _reference_pair()
    ids = torch.randint(0, 60000, (2, 16))
    state = torch.randn(2, 16, 96) * 0.5
    a = ours(ids, input_states=state, num_steps=3, labels=ids)
    b = theirs(ids, input_states=state, num_steps=3, labels=ids)
    assert torch.allclose(a.logits, b.logits, rtol=1e-4, atol=1e-4)
    assert torch.allclose(a.loss, b.loss, rtol=1e-5) and torch.allclose(a.latent_states, b.latent_states, atol=1e-4)
    # prefill + token-by-token decoding through the per-step cache
    oa = ours(ids[:, :10], num_steps=3, init_scale=0.0, use_cache=True)
    ob = theirs(ids[:, :10], num_steps=3, init_scale=0.0, use_cache=True,
                past_key_values=mod.HuginnDynamicCache(), cache_position=torch.arange(10))
    assert torch.allclose(oa.logits, ob.logits, rtol=1e-4, atol=1e-4)
    for t in range(10, 16):
        pos = torch.tensor([t])
        oa = ours(ids[:, t:t + 1], num_steps=3, init_scale=0.0, use_cache=True, past_key_values=oa.past_key_values,
                  cache_position=pos)
        ob = theirs(ids[:, t:t + 1], num_steps=3, init_scale=0.0, use_cache=True, past_key_values=ob.past_key_values,
                    cache_position=pos)
        assert torch.allclose(oa.logits, ob.logits, rtol=1e-4, atol=2e-4), t
    assert oa.past_key_values.get_seq_length() == 16
    assert abs(oa.past_key_values.get_memory_usage() - ob.past_key_values.get_memory_usage()) < 1e-6


@needs_ref
def test_kl_exit_hand_loop_matches_reference_primitives():
    ours, theirs, mod = _reference_pair()
    ids = torch.randint(0, 60000, (1, 9))
    traces = []
    for model, evaluator, cache in ((ours, get_adaptive_exit_evaluator(ours, "kl", 5e-4), RecurrentKVCache()),
                                    (theirs, mod.get_adaptive_exit_evaluator(theirs, "kl", 5e-4),
                                     mod.HuginnDynamicCache())):
        aux = dict(past_key_values=cache, cache_position=torch.arange(9))
        e, block_idx = model.embed_inputs(ids, **aux)
        x = torch.zeros_like(e)
        evaluator.init(x)
        vals = []
        for step in range(6):
            x, block_idx, _ = model.iterate_one_step(e, x, block_idx=block_idx, **aux, current_step=step)
            exits, out, v = evaluator.check(model, x, aux)
            vals.append(float(v[0]))
        traces.append((vals, out.logits))
    assert traces[0][0] == pytest.approx(traces[1][0], rel=1e-3, abs=1e-6)
    assert torch.allclose(traces[0][1], traces[1][1], rtol=1e-4, atol=2e-4)


@needs_ref
@pytest.mark.parametrize("strategy", ["latest-m4", "available-m4", "always-last-m4", "skip", "latest-m4-compress-s4",
                                      "latest-m4-compress-anchor"])
def test_cache_lookup_strategies_match_reference(strategy):
    mod = refload.module("raven_modeling_minimal")
    torch.manual_seed(1)
    a, b = RecurrentKVCache(strategy), mod.HuginnDynamicCache(strategy)
    depth_per_token = [3, 1, 2, 3, 1]  # recurrences computed for each position (ragged depth)
    for pos, depth in enumerate(depth_per_token):
        steps = [0, 1] + [2 + 4 * j + blk for j in range(depth) for blk in range(4)] + [-1, -2]
        for s in steps:
            k, v = torch.randn(1, 1, 2, 8), torch.randn(1, 1, 2, 8)
            ka, va = a.update(k, v, s)
            kb, vb = b.update(k.transpose(1, 2), v.transpose(1, 2), torch.tensor(s))
            assert torch.equal(ka.transpose(1, 2), kb) and torch.equal(va.transpose(1, 2), vb), (pos, s)
    a.clear_last_k_entries(2)
    b.clear_last_k_entries(2)
    assert a.get_seq_length() == b.get_seq_length() == 3
    assert abs(a.get_memory_usage() - b.get_memory_usage()) < 1e-9


def test_training_model_converts_to_inference_model():
    torch.manual_seed(2)
    cfg = ModelConfig.from_name("tiny-raven-cpu")
    train_model = cfg.construct_model().eval()
    hf = RavenForCausalLM.from_training_model(train_model).eval()
    ids = torch.randint(0, 8192, (2, 32))
    state = torch.zeros(2, 32, 256)
    with torch.no_grad():
        a = train_model(ids, return_logits=True, num_steps_pair=torch.tensor([3, 0]), input_states=state)["logits"]
        b = hf(ids, input_states=state, num_steps=3).logits
    assert torch.allclose(a, b, rtol=1e-4, atol=1e-4)
    assert set(hf.state_dict()) == set(train_model.state_dict())


def test_generate_paths_and_dispatch(tmp_path):
    m = _ours(3)
    ids = torch.randint(0, 60000, (2, 10))
    plain = m.generate(ids, max_new_tokens=6, num_steps=4, init_scale=0.0)
    assert plain.shape == (2, 16) and torch.equal(plain[:, :10], ids)
    # adaptive compute with a threshold nobody reaches equals fixed-depth decoding and reports the step counts
    out = m.generate(ids, max_new_tokens=6, num_steps=4, init_scale=0.0, criterion="kl", exit_threshold=0.0,
                     generation_config=_cfg(return_dict_in_generate=True))
    assert torch.equal(out.sequences, plain) and out.scores["compute_steps"][0] == [4, 4]
    early = m.generate(ids, max_new_tokens=3, num_steps=8, init_scale=0.0, criterion="latent-diff", exit_threshold=10.0,
                       generation_config=_cfg(return_dict_in_generate=True), cache_lookup_strategy="latest-m4")
    assert early.scores["compute_steps"][0] == [1, 1]  # everything exits after the first recurrence
    spec = m.generate(ids, max_new_tokens=6, draft_steps=2, lookahead_for_draft=3, num_steps=4, init_scale=0.0)
    assert torch.equal(spec[:, :16], plain)  # greedy speculative decoding reproduces greedy decoding
    cont = m.generate(ids, max_new_tokens=4, num_steps=4, init_scale=0.0, continuous_compute=True)
    assert cont.shape == (2, 14)
    diff = m.generate(ids[:1], max_new_tokens=4, headway=2, inner_recurrence=2, num_steps=4, init_scale=0.0)
    assert diff.shape[0] == 1 and 10 < diff.shape[1] <= 14
    sampled = m.generate(ids, max_new_tokens=3, num_steps=2, generation_config=_cfg(do_sample=True, temperature=0.7,
                                                                                   top_k=50, top_p=0.9, min_p=0.01,
                                                                                   repetition_penalty=1.2))
    assert sampled.shape == (2, 13)
    m.save_pretrained(str(tmp_path))
    again = RavenForCausalLM.from_pretrained(str(tmp_path)).eval()
    assert torch.equal(again.generate(ids, max_new_tokens=6, num_steps=4, init_scale=0.0), plain)


def _cfg(**kw):
    from types import SimpleNamespace

    return SimpleNamespace(**kw)


def test_legacy_model_returns_attention_maps():
    from recurrent_pretraining_b200.models import legacy
    from recurrent_pretraining_b200.models.hf_config import RavenConfig

    torch.manual_seed(0)
    cfg = RavenConfig(n_embd=64, n_heads=4, n_layers=4, block_size=32, vocab_size=128, intermediate_size=96,
                      n_layers_in_recurrent_block=2, n_layers_in_prelude=1, n_layers_in_coda=1, mean_recurrence=2)
    model = legacy.RavenForCausalLM(cfg).eval()
    ids = torch.randint(0, 128, (2, 12))
    states = torch.zeros(2, 12, 64)
    with torch.no_grad():
        plain = model(ids, input_states=states, num_steps=2)
        out = model(ids, input_states=states, num_steps=2, output_details={"return_attention": True})
    assert plain.attention_maps is None
    assert torch.allclose(plain.logits, out.logits, atol=1e-4)
    assert set(out.attention_maps) == {0, 1, 2, 3, 4, -1}  # prelude 0, two recurrences of two blocks, coda
    m = out.attention_maps[0]
    assert m.shape == (2, 12, 12) and float(m.triu(1).abs().max()) == 0.0 and float(m[:, 0, 0].min()) == 1.0


def test_forward_with_adaptive_compute_per_position():
    from recurrent_pretraining_b200.models.exit_criteria import KLExitEvaluator, NoOpExitEvaluator
    from recurrent_pretraining_b200.models.hf import RavenForCausalLM
    from recurrent_pretraining_b200.models.hf_config import RavenConfig

    torch.manual_seed(0)
    cfg = RavenConfig(n_embd=64, n_heads=4, n_layers=4, block_size=32, vocab_size=128, intermediate_size=96,
                      n_layers_in_recurrent_block=2, n_layers_in_prelude=1, n_layers_in_coda=1, mean_recurrence=5)
    model = RavenForCausalLM(cfg).eval()
    ids = torch.randint(0, 128, (1, 7))
    # without an exit every position runs the full depth and the result equals the ordinary (parallel) forward
    full = model.forward_with_adaptive_compute(ids, NoOpExitEvaluator(), init_scale=0.0)
    assert full.stats["compute_steps"] == [5] * 7
    want = model(ids, num_steps=5, init_scale=0.0).logits
    assert torch.allclose(full.logits, want, atol=2e-4), (full.logits - want).abs().max()
    out = model.forward_with_adaptive_compute(ids, KLExitEvaluator(model, exit_threshold=1e9), labels=ids)
    assert out.stats["compute_steps"] == [1] * 7 and torch.isfinite(out.loss)  # the first check already fires


def test_legacy_surface_old_signatures_and_helpers():
    from recurrent_pretraining_b200.models import legacy
    from recurrent_pretraining_b200.models.hf_config import RavenConfig
    from recurrent_pretraining_b200.ops import reference as ref

    torch.manual_seed(0)
    cfg = RavenConfig(n_embd=64, n_heads=4, n_layers=4, block_size=32, vocab_size=128, intermediate_size=96,
                      n_layers_in_recurrent_block=2, n_layers_in_prelude=1, n_layers_in_coda=1, mean_recurrence=2)
    model = legacy.RavenForCausalLM(cfg).eval()
    e = torch.randn(2, 5, 64)
    assert float(model.initialize_state(e, deterministic=True).abs().sum()) == 0.0
    assert model.initialize_state(e).shape == e.shape and float(model.initialize_state(e, 0.0).abs().sum()) == 0.0
    fc = legacy.precompute_freqs_cis(16, 5, 50000.0)
    assert fc.shape == (1, 5, 1, 8, 2)
    q, k = torch.randn(2, 5, 4, 16), torch.randn(2, 5, 4, 16)
    rq, rk = legacy.apply_rotary_emb_complex_like(q, k, fc)
    cos, sin = ref.rope_tables(16, 5, 50000.0)
    assert torch.allclose(rq, ref.rope_interleaved(q, cos, sin)) and rk.shape == k.shape
    y, amap = model.compute_eager_sdpa(q.transpose(1, 2), k.transpose(1, 2), k.transpose(1, 2))
    want = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), k.transpose(1, 2),
                                                            is_causal=True)
    assert torch.allclose(y, want, atol=1e-5) and amap.shape == (2, 5, 5)
    st = model.get_stats(torch.randn(2, 5, 128), e, e + 0.1, None, e, 3, 1)
    assert st["entropy"].shape == (2, 5) and st["num_steps_no_grad"] == 3 and float(st["rel_residual"].max()) < 1.0
    assert legacy.SandwichBlock.__name__ == "SandwichBlock" and legacy.RMSNorm.__name__ == "RMSNorm"
    legacy.register_auto_classes()
    cache = legacy.HuginnDynamicCache()
    cache.reset()
    assert cache.get_seq_length() == 0


def test_padding_mask_is_optional_and_hides_padding_when_on():
    """``compile_mask``: causal + padding keys hidden + optional custom mask.  Off by default (the reference's forward
    builds no mask); when on, a left-padded row gives the logits of the unpadded row, and a custom [B, Sq, Sk] mask
    changes exactly the rows it restricts."""
    model = _ours()
    PAD = 65509
    torch.manual_seed(1)
    row = torch.randint(0, 1000, (1, 10))
    padded = torch.cat([torch.full((1, 6), PAD), row], 1)
    with torch.no_grad():
        plain = model(row, num_steps=3, init_scale=0.0).logits
        off = model(padded, num_steps=3, init_scale=0.0).logits[:, 6:]
        model.apply_padding_mask = True
        on = model(padded, num_steps=3, init_scale=0.0).logits[:, 6:]
        mask = model.compile_mask(padded)
        assert mask.shape == (1, 1, 16, 16) and not mask[0, 0, :, :6].any() and mask[0, 0, 15, 6:].all()
        assert model.compile_mask(row) is None                                     # nothing to hide
        assert model.compile_mask(padded[:, -1:], past_key_values=object()) is None  # single-token step on a cache
        am = torch.ones(1, 10, 10, dtype=torch.bool).tril()
        am[0, 7:, 2] = False                                                      # queries 7.. may not see key 2
        restricted = model(row, attention_mask=am, num_steps=3, init_scale=0.0).logits
    assert (on - plain).abs().max().item() < 1e-4          # padding hidden: same as the unpadded row
    assert (off - plain).abs().max().item() > 1e-3         # default (reference behaviour): padding is attended to
    assert (restricted[:, :7] - plain[:, :7]).abs().max().item() < 1e-5
    assert (restricted[:, 7:] - plain[:, 7:]).abs().max().item() > 1e-4


def test_static_cache_gives_the_dynamic_cache_logits():
    """Prefill + token-by-token decoding on the preallocated cache equals the same on the dynamic cache (lookup ``full``
    and the folded ``compress-s4`` form)."""
    from recurrent_pretraining_b200.models.kv_cache import HuginnStaticCache, StaticRecurrentCache

    assert HuginnStaticCache is StaticRecurrentCache
    model = _ours()
    cfg = model.config
    steps = 5
    torch.manual_seed(2)
    ids = torch.randint(0, 1000, (2, 9))
    for strategy in ("full", "compress-s4"):
        dyn = RecurrentKVCache(strategy)
        sta = StaticRecurrentCache(max_length=16, max_num_steps=4 + 4 * steps, num_heads=cfg.num_key_value_heads,
                                   hidden_dim=cfg.n_embd // cfg.num_attention_heads, batch_size=2,
                                   lookup_strategy=strategy)
        with torch.no_grad():
            for cache in (dyn, sta):
                out = model(ids[:, :6], num_steps=steps, init_scale=0.0, past_key_values=cache, use_cache=True)
                rows = [out.logits[:, -1]]
                for t in range(6, 9):
                    out = model(ids[:, t:t + 1], num_steps=steps, init_scale=0.0, past_key_values=cache, use_cache=True,
                                cache_position=torch.tensor([t]))
                    rows.append(out.logits[:, -1])
                cache.result = torch.stack(rows, 1)
        assert (dyn.result - sta.result).abs().max().item() < 1e-4, strategy
        assert sta.get_seq_length() == 9 and sta.get_memory_usage() > 0
    sta.reset()
    assert sta.get_seq_length() == 0 and not sta.valid_mask.any()


def test_diffusion_style_sampler_strategies_statistics_and_analysis_tablets():
    """Every freeze strategy of the wavefront sampler runs within its length budget; with no randomness in the state
    (init_scale 0, no noise mixing, no embedding EMA) the run is repeatable; the summary carries the reference's counter
    names and the analysis tablets have one row per sweep."""
    from transformers import GenerationConfig

    m = _ours(5)
    torch.manual_seed(0)
    ids = torch.randint(0, 60000, (1, 10))
    gc = GenerationConfig(max_new_tokens=6, do_sample=False, return_dict_in_generate=True)   # no max_length given
    kw = dict(generation_config=gc, init_scale=0.0, ema_embeds=0.0, state_noise_mixing=0.0, inner_recurrence=2,
              num_steps=4, exit_t=0.5)
    seen = {}
    for strategy in ("latent-diff", "latent-acceleration-1", "latent-acceleration-2", "token-stability", "fixed"):
        for headway in (1, 2):
            out = m.generate_diffusion_style(ids, freeze_strategy=strategy, headway=headway, **kw)
            seq = out.sequences
            assert seq.shape[0] == 1 and 10 < seq.shape[1] <= 16 and torch.equal(seq[:, :10], ids), (strategy, headway)
            for key in ("num_core_forward_passes", "num_tokens_forward", "num_cache_clears", "num_standing_waves",
                        "diffusion_steps", "gen_seq_length", "len_prefill", "recurrence_per_position",
                        "token_stable_per_position"):
                assert key in out.scores, key
            assert out.scores["len_prefill"] == 10 and out.scores["num_core_forward_passes"] == \
                2 * out.scores["diffusion_steps"]
            assert out.scores["recurrence_per_position"].shape == (1, seq.shape[1]) or \
                out.scores["recurrence_per_position"].shape[1] >= seq.shape[1]
            seen[(strategy, headway)] = seq
    again = m.generate_diffusion_style(ids, freeze_strategy="latent-acceleration-2", headway=2, **kw)
    assert torch.equal(again.sequences, seen[("latent-acceleration-2", 2)])
    with pytest.raises(ValueError):
        m.generate_diffusion_style(ids, freeze_strategy="latent-nonsense", **kw)
    narrow = m.generate_diffusion_style(ids, freeze_strategy="token-stability", headway=3, max_wavefront=4, **kw)
    assert narrow.scores["num_standing_waves"] > 0
    full = m.generate_diffusion_style(ids, freeze_strategy="latent-diff", headway=2, return_analysis_tablets=True,
                                      return_full_state_tablet=True, **kw)
    tab = full.hidden_states
    steps = tab["last_step"]
    assert steps == full.scores["diffusion_steps"] and tab["last_recurrence"] == 2 * steps
    assert tab["token_tablet"].shape == tab["frozen_tablet"].shape == tab["counter_tablet"].shape
    assert tab["state_tablet"].dtype == torch.bfloat16 and tab["state_tablet"].shape[:2] == tab["token_tablet"].shape
    used = min(steps, tab["token_tablet"].shape[0])
    assert bool((tab["token_tablet"][:used, :10] == ids[0]).all())             # every sweep starts from the prompt
    assert int(tab["token_tablet"][used:].abs().sum()) == 0                      # rows past the last sweep stay empty
    assert int(tab["counter_tablet"][used - 1].max()) >= 4


@needs_ref
def test_fresh_inference_model_is_initialised_like_the_reference():
    """A newly constructed HF-style model: same parameter names and per-tensor deviations as the reference's
    ``_init_weights`` gives -- in particular the up half of every gated-MLP input projection is drawn with the
    output-projection deviation (the training model uses the input deviation for both halves)."""
    mod = refload.module("raven_modeling_minimal")
    cfgmod = refload.module("raven_config_minimal")
    mod.RavenForCausalLM._tied_weights_keys = {"lm_head.weight": "transformer.wte.weight"}
    torch.manual_seed(0)
    theirs = dict(mod.RavenForCausalLM(cfgmod.RavenConfig(**SMALL)).named_parameters())
    torch.manual_seed(0)
    ours = dict(RavenForCausalLM(RavenConfig(**SMALL)).named_parameters())
    assert set(theirs) == set(ours)
    for name, want in theirs.items():
        got = ours[name]
        assert got.shape == want.shape
        parts = [slice(None)]
        if name.endswith("mlp.fc.weight"):
            half = want.shape[0] // 2
            parts = [slice(0, half), slice(half, None)]
        for part in parts:
            a, b = float(want[part].float().std()), float(got[part].float().std())
            assert abs(a - b) <= 0.06 * max(a, 1e-9), (name, a, b)
