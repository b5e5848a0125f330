"""Named model shapes.

The shape names and their numeric values are the public contract shared with the
reference registry (recpre/model_registry.py:13-787): a user can ask for
``nebel-raven-3.5b`` and get the same widths, head counts, layer split and recurrence
settings.  The table here is stored as *families* (a base dict plus per-model deltas)
and is expanded on import into ``name_to_config``.
"""
from __future__ import annotations

from copy import deepcopy

_ORG = "tomg-group-umd"


def _hf(name: str, org: str = _ORG) -> dict:
    return {"org": org, "name": name}


# --------------------------------------------------------------------------------------
# family bases
# --------------------------------------------------------------------------------------
_LLAMA_LIKE = dict(
    architecture_class_name="GPT",
    bias=False,
    norm_class_name="RMSNorm_llama",
    norm_eps=1e-5,
    mlp_class_name="GatedMLP",
    nonlin_name="SiLU",
    init_strategy="scaled",
    vocab_size=32000,
    padding_multiple=4096,
    block_size=4096,
)

_RAVEN = dict(
    architecture_class_name="RecurrentGPT",
    block_size=4096,
    vocab_size=65536,
    padding_multiple=4096,
    tie_embeddings=True,
    bias=False,
    block_class_name="TransformerPostNormBlock",
    norm_class_name="RMSNorm_llama",
    norm_eps=1e-5,
    mlp_class_name="GatedMLP",
    nonlin_name="SiLU",
    init_strategy="scaled",
    init_orthogonal=True,
    state_init="like-init",
    injection_type="add",
    sampling_scheme="poisson-fill",
    n_layers_in_recurrent_block=4,
    n_layers_in_prelude=1,
    n_layers_in_coda=1,
)

_RAVEN_35 = dict(
    _RAVEN,
    num_attention_heads=55,
    num_key_value_heads=55,
    n_embd=5280,
    intermediate_size=17920,
    norm_eps=1e-6,
    mean_recurrence=32,
    mean_backprop_depth=8,
    n_layers_in_prelude=2,
    n_layers_in_coda=2,
    sampling_scheme="poisson-lognormal-filling",
)

_TINY_LLAMA = dict(
    architecture_class_name="GPT",
    block_size=2048,
    vocab_size=32000,
    padding_multiple=4096,
    num_attention_heads=32,
    num_key_value_heads=4,
    bias=False,
    norm_class_name="RMSNorm",
    norm_eps=1e-5,
    mlp_class_name="GatedMLP",
    nonlin_name="SiLU",
)

_GEMMA = dict(
    architecture_class_name="GPT",
    scale_embeddings=True,
    vocab_size=50304,
    block_size=8192,
    bias=False,
    norm_class_name="RMSNorm",
    mlp_class_name="GatedMLP",
    nonlin_name="GELU",
)


def _mk(base: dict, name: str, hf_name: str | None = None, hf_org: str = _ORG, **delta) -> dict:
    d = deepcopy(base)
    d.update(delta)
    d["name"] = name
    d["hf_config"] = _hf(hf_name or name, hf_org)
    return d


configs: list[dict] = [
    # ---- non-recurrent baselines (recpre/model_registry.py:13-91) ----
    _mk(_LLAMA_LIKE, "baby-llama-200m", padding_multiple=32768, n_layer=12, num_attention_heads=32,
        num_key_value_heads=8, n_embd=1024, intermediate_size=2816),
    _mk(_LLAMA_LIKE, "baby-llama-long-200m", n_layer=24, num_attention_heads=32, num_key_value_heads=8,
        n_embd=768, intermediate_size=2048),
    _mk(_LLAMA_LIKE, "baby-snake-200m", hf_name="baby-llama-long-200m", n_layer=48, num_attention_heads=32,
        num_key_value_heads=8, n_embd=512, intermediate_size=1536),
    _mk(_LLAMA_LIKE, "gpt2-124m", block_size=1024, n_layer=12, num_attention_heads=12, num_key_value_heads=12,
        n_embd=768, intermediate_size=3072, norm_class_name="LayerNorm", mlp_class_name="BaseMLP",
        nonlin_name="GELU"),
    # ---- pure-GEMM sanity models (recpre/model_registry.py:97-136) ----
    dict(name="brick-200m", hf_config=_hf("brick-200m"), architecture_class_name="GPT", block_size=4096,
         vocab_size=32000, padding_multiple=4096, n_layer=4, n_embd=2048, bias=False,
         norm_class_name="Identity", norm_eps=1e-5, mlp_class_name="BaseMLP", nonlin_name="ReLU",
         intermediate_size=8192, init_strategy="normal", attn_impl="debug-skip"),
    dict(name="big-brick-200m", hf_config=_hf("big-brick-200m"), architecture_class_name="GPT", block_size=4096,
         vocab_size=32000, padding_multiple=4096, n_layer=24, n_embd=4096, bias=False,
         block_class_name="Brick", mlp_class_name="BrickLP", nonlin_name="ReLU", intermediate_size=4096,
         init_strategy="normal", attn_impl="debug-skip"),
    # ---- recurrent family (recpre/model_registry.py:169-488) ----
    _mk(_RAVEN, "baby-recurrent-200m", vocab_size=32000, num_attention_heads=32, num_key_value_heads=8,
        n_embd=1024, intermediate_size=2816, mean_recurrence=20, mean_backprop_depth=4,
        tie_embeddings=False, sampling_scheme="poisson-unbounded"),
    _mk(_RAVEN, "debug-recurrent", hf_name="baby-recurrent-200m", block_size=384, vocab_size=32000,
        num_attention_heads=16, num_key_value_heads=8, n_embd=256, intermediate_size=256,
        init_orthogonal=False, n_layers_in_recurrent_block=2, mean_recurrence=2, mean_backprop_depth=1,
        tie_embeddings=False, sampling_scheme="poisson-unbounded"),
    _mk(_RAVEN, "magpie-150m", num_attention_heads=32, num_key_value_heads=32, n_embd=1024,
        intermediate_size=3520, mean_recurrence=20, mean_backprop_depth=4),
    _mk(_RAVEN, "corax-raven-800m", num_attention_heads=32, num_key_value_heads=32, n_embd=4096,
        intermediate_size=8192, n_layers_in_recurrent_block=2, mean_recurrence=20, mean_backprop_depth=4),
    _mk(_RAVEN, "kolk-raven-1.1b", num_attention_heads=64, num_key_value_heads=64, n_embd=4096,
        intermediate_size=8192, mean_recurrence=24, mean_backprop_depth=8),
    _mk(_RAVEN, "tower-raven-3b", num_attention_heads=64, num_key_value_heads=64, n_embd=4096,
        intermediate_size=8192, n_layers_in_recurrent_block=8, mean_recurrence=32, mean_backprop_depth=8,
        n_layers_in_prelude=2, n_layers_in_coda=2),
    _mk(_RAVEN, "deluge-raven-4b", hf_name="merseburg-raven-4b", num_attention_heads=64, num_key_value_heads=64,
        n_embd=7040, intermediate_size=14080, mean_recurrence=32, mean_backprop_depth=8,
        n_layers_in_prelude=2, n_layers_in_coda=2),
    _mk(_RAVEN_35, "merseburg-raven-3.5b", block_class_name="SandwichBlock",
        norm_class_name="UnparametrizedRMSNorm", qk_bias=False),
    _mk(_RAVEN_35, "corone-raven-3.5b", hf_name="merseburg-raven-3.5b", block_class_name="TransformerPreNormBlock",
        init_strategy="takase", init_orthogonal=False, injection_type="linear", qk_bias=True,
        activation_checkpoint_impl="per-iteration"),
    # the flagship: 3,564,976,800 parameters, 1,581,592,320 of them in the recurrent core
    _mk(_RAVEN_35, "nebel-raven-3.5b", block_class_name="SandwichBlock", init_strategy="takase",
        init_orthogonal=False, injection_type="linear", qk_bias=True,
        activation_checkpoint_impl="per-iteration"),
    # ---- small llama / gemma shapes (recpre/model_registry.py:526-784) ----
    dict(name="Llama-debug", hf_config=_hf("Llama-debug"), architecture_class_name="GPT", vocab_size=32000,
         block_size=384, num_attention_heads=8, num_key_value_heads=2, n_embd=512, padding_multiple=4096,
         n_layer=4, bias=False, norm_class_name="RMSNorm", mlp_class_name="GatedMLP", nonlin_name="SiLU",
         intermediate_size=256),
    _mk(_TINY_LLAMA, "tiny-llama-190m", n_layer=12, n_embd=1024, intermediate_size=2816),
    _mk(_TINY_LLAMA, "tiny-llama-1.1b", hf_name="TinyLlama-1.1B-intermediate-step-1431k-3T", hf_org="TinyLlama",
        n_layer=22, n_embd=2048, intermediate_size=5632),
    _mk(_TINY_LLAMA, "tiny-llama-1.1b-chat", hf_name="TinyLlama-1.1B-Chat-v1.0", hf_org="TinyLlama",
        n_layer=22, n_embd=2048, intermediate_size=5632),
    _mk(_GEMMA, "PyGemma-2-2b", hf_name="gemma-2-2b", hf_org="google", intermediate_size=8192, n_embd=2048,
        n_layer=26, num_attention_heads=16, num_key_value_heads=8),
    _mk(_GEMMA, "PyGemma-2-1b", hf_name="gemma-2-2b", hf_org="google", intermediate_size=8192, n_embd=2048,
        n_layer=12, num_attention_heads=16, num_key_value_heads=8),
    _mk(_GEMMA, "PyGemma-2-500m", hf_name="gemma-2-2b", hf_org="google", intermediate_size=6144, n_embd=1536,
        n_layer=12, num_attention_heads=12, num_key_value_heads=6),
    _mk(_GEMMA, "PyGemma-2-100m", hf_name="gemma-2-2b", hf_org="google", intermediate_size=3072, n_embd=768,
        n_layer=3, num_attention_heads=6, num_key_value_heads=3),
    # ---- shapes added by this framework (plumbing test and kernel bring-up) ----
    # tiny CPU/gloo model: 256 wide, 4 heads x 64, prelude 1 / core 2 / coda 1, SwiGLU 704, vocab 8192
    _mk(_RAVEN_35, "tiny-raven-cpu", block_size=256, vocab_size=8192, padding_multiple=512, n_embd=256,
        num_attention_heads=4, num_key_value_heads=4, intermediate_size=704, block_class_name="SandwichBlock",
        init_strategy="takase", init_orthogonal=False, injection_type="linear", qk_bias=True,
        n_layers_in_recurrent_block=2, n_layers_in_prelude=1, n_layers_in_coda=1, mean_recurrence=4,
        mean_backprop_depth=2),
    # small GPU smoke shape that keeps the flagship's awkward factors (hd 96, width not a power of two)
    _mk(_RAVEN_35, "smoke-raven-96", block_size=512, vocab_size=4096, padding_multiple=512, n_embd=480,
        num_attention_heads=5, num_key_value_heads=5, intermediate_size=1280, block_class_name="SandwichBlock",
        init_strategy="takase", init_orthogonal=False, injection_type="linear", qk_bias=True,
        n_layers_in_recurrent_block=2, n_layers_in_prelude=1, n_layers_in_coda=1, mean_recurrence=4,
        mean_backprop_depth=2),
]

name_to_config: dict[str, dict] = {c["name"]: c for c in configs}


def lookup(name: str) -> dict:
    """Return a *copy* of the registry dict for ``name`` (also matches ``hf_config.name``)."""
    if name in name_to_config:
        return deepcopy(name_to_config[name])
    for c in configs:
        if c["hf_config"]["name"] == name:
            return deepcopy(c)
    raise ValueError(f"{name!r} is not a supported config name")
