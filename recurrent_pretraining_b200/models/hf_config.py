"""``RavenConfig``: the Hugging Face configuration of the inference/finetune model (``model_type = huginn_raven``).

Field names and defaults follow recpre/raven_config_minimal.py:7-98 so that a ``config.json`` written by either
implementation loads in the other.
"""
from __future__ import annotations

import math

from transformers import PretrainedConfig


class RavenConfig(PretrainedConfig):
    model_type = "huginn_raven"
    keys_to_ignore_at_inference = [""]
    attribute_map = {"num_attention_heads": "n_heads", "hidden_size": "n_embd", "num_hidden_layers": "n_layers"}

    def __init__(self, n_embd: int = 5280, n_heads: int = 55, n_layers: int = 8, block_size: int = 4096,
                 vocab_size: int = 65536, padding_multiple: int = 4096, tie_embeddings: bool = True,
                 intermediate_size: int = 17920, bias: bool = False, architecture_class_name: str = "RecurrentGPT",
                 block_class_name: str = "SandwichBlock", norm_class_name: str = "RMSNorm_llama", norm_eps: float = 1e-6,
                 mlp_class_name: str = "GatedMLP", nonlin_name: str = "SiLU", init_strategy: str = "takase",
                 init_orthogonal: bool = False, state_init: str = "like-init", injection_type: str = "linear",
                 n_layers_in_recurrent_block: int = 4, mean_recurrence: int = 32, sampling_scheme: str =
                 "poisson-lognormal-filling", mean_backprop_depth: int = 8, n_layers_in_prelude: int = 2,
                 n_layers_in_coda: int = 2, qk_bias: bool = True, activation_checkpoint_impl: str = "per-iteration",
                 rope_base: float = 50_000, torch_dtype: str = "bfloat16", transformers_version: str = "4.47.1",
                 **kwargs):
        self.n_embd, self.n_heads, self.n_layers = n_embd, n_heads, n_layers
        self.block_size, self.vocab_size = block_size, vocab_size
        self.padding_multiple = padding_multiple
        self.padded_vocab_size = vocab_size
        self.tie_embeddings = tie_embeddings
        self.intermediate_size = intermediate_size
        self.bias = bias
        self.architecture_class_name = architecture_class_name
        self.block_class_name = block_class_name
        self.norm_class_name = norm_class_name
        self.norm_eps = norm_eps
        self.mlp_class_name = mlp_class_name
        self.nonlin_name = nonlin_name
        self.init_strategy = init_strategy
        self.init_orthogonal = init_orthogonal
        self.state_init = state_init
        self.injection_type = injection_type
        self.n_layers_in_recurrent_block = n_layers_in_recurrent_block
        self.mean_recurrence = mean_recurrence
        self.sampling_scheme = sampling_scheme
        self.mean_backprop_depth = mean_backprop_depth
        self.n_layers_in_prelude = n_layers_in_prelude
        self.n_layers_in_coda = n_layers_in_coda
        self.qk_bias = qk_bias
        self.activation_checkpoint_impl = activation_checkpoint_impl
        self.rope_base = rope_base
        self.tie_word_embeddings = tie_embeddings
        # runtime attributes
        self.num_key_value_heads = n_heads
        self.head_dim = n_embd // n_heads
        self.effective_expected_depth = n_layers_in_prelude + n_layers_in_coda + n_layers_in_recurrent_block * mean_recurrence
        self.init_values = {"std": math.sqrt(2 / (5 * n_embd)),
                            "out_proj": math.sqrt(2 / (5 * n_embd)) / math.sqrt(2 * self.effective_expected_depth),
                            "embedding": math.sqrt(2 / (5 * n_embd)), "embed_scale": math.sqrt(n_embd)}
        self.test_time_noise = kwargs.pop("test_time_noise", 0)
        self.test_time_noise_type = kwargs.pop("test_time_noise_type", "fixed")
        for derived in ("tie_word_embeddings", "padded_vocab_size", "num_key_value_heads", "head_dim",
                        "effective_expected_depth", "init_values"):
            kwargs.pop(derived, None)
        super().__init__(tie_word_embeddings=tie_embeddings, **kwargs)

    # ---- bridge to the training-side config ---------------------------------------------------------
    @classmethod
    def from_model_config(cls, mc) -> "RavenConfig":
        return cls(n_embd=mc.n_embd, n_heads=mc.n_head, n_layers=mc.n_layers_in_prelude + mc.n_layers_in_coda +
                   mc.n_layers_in_recurrent_block, block_size=mc.block_size, vocab_size=mc.padded_vocab_size,
                   padding_multiple=mc.padding_multiple, tie_embeddings=mc.tie_embeddings,
                   intermediate_size=mc.intermediate_size, bias=mc.bias, block_class_name=mc.block_class_name,
                   norm_class_name=mc.norm_class_name, norm_eps=mc.norm_eps, mlp_class_name=mc.mlp_class_name,
                   nonlin_name=mc.nonlin_name, init_strategy=mc.init_strategy, init_orthogonal=mc.init_orthogonal,
                   state_init=mc.state_init, injection_type=mc.injection_type,
                   n_layers_in_recurrent_block=mc.n_layers_in_recurrent_block, mean_recurrence=mc.mean_recurrence,
                   sampling_scheme=mc.sampling_scheme, mean_backprop_depth=mc.mean_backprop_depth,
                   n_layers_in_prelude=mc.n_layers_in_prelude, n_layers_in_coda=mc.n_layers_in_coda,
                   qk_bias=mc.qk_bias, rope_base=mc.rope_settings.rope_base)

    def to_model_config(self):
        """The equivalent training-side ``ModelConfig`` (used to build the shared block modules)."""
        from ..config import ModelConfig, RoPESettings

        return ModelConfig(
            name="raven-hf", architecture_class_name="RecurrentGPT", block_size=self.block_size, n_embd=self.n_embd,
            intermediate_size=self.intermediate_size, num_attention_heads=self.n_heads,
            num_key_value_heads=self.num_key_value_heads, vocab_size=self.vocab_size, padding_multiple=1,
            padded_vocab_size=self.vocab_size, rope_settings=RoPESettings(rope_base=self.rope_base),
            block_class_name=self.block_class_name, norm_class_name=self.norm_class_name, norm_eps=self.norm_eps,
            mlp_class_name=self.mlp_class_name, nonlin_name=self.nonlin_name, bias=self.bias, qk_bias=self.qk_bias,
            init_strategy=self.init_strategy, init_orthogonal=self.init_orthogonal, injection_type=self.injection_type,
            n_layers_in_recurrent_block=self.n_layers_in_recurrent_block, n_layers_in_prelude=self.n_layers_in_prelude,
            n_layers_in_coda=self.n_layers_in_coda, state_init=self.state_init, sampling_scheme=self.sampling_scheme,
            mean_recurrence=self.mean_recurrence, mean_backprop_depth=self.mean_backprop_depth,
            tie_embeddings=self.tie_embeddings)
