"""HF-compatible inference / finetuning model: ``RavenForCausalLM``.

Public surface kept from recpre/raven_modeling_minimal.py:542-2323: ``forward(input_ids, input_embeds, input_states,
attention_mask, position_ids, labels, num_steps, past_key_values, output_details, use_cache, cache_position,
init_scale)`` returning ``CausalLMOutputRecurrentLatents``; the building blocks ``embed_inputs``, ``iterate_one_step``,
``predict_from_latents``, ``initialize_state``; the ``generate`` dispatcher with the minimal, adaptive-compute,
speculative and diffusion-style samplers (``models/generation.py``); the per-recurrence-step KV cache and its lookup
strategies (``models/kv_cache.py``); the exit criteria (``models/exit_criteria.py``).  State-dict keys are identical to
the training model, so checkpoints move between the two without renaming.

The modules are the same block classes the training model uses; all arithmetic goes through ``ops.functional`` and
runs the sm_100a kernels on a GPU.  The native decode engine (``engine/decode.py``) drives this model's weights with
CUDA graphs for serving; ``generate`` here is the reference-faithful eager path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Union

import torch
import torch.nn as nn
import torch.utils.checkpoint
from transformers import GenerationMixin, PreTrainedModel
from transformers.utils import ModelOutput

from ..ops import functional as ops
from ..ops import reference as ref
from .blocks import Linear, make_block, make_norm
from .generation import RavenGenerationMixin
from .hf_config import RavenConfig
from .kv_cache import RecurrentKVCache


@dataclass
class CausalLMOutputRecurrentLatents(ModelOutput):
    loss: Optional[torch.Tensor] = None
    log_ppl: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    past_key_values: Optional[object] = None
    latent_states: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None
    attention_maps: Optional[dict] = None
    stats: Optional[dict] = None


_DEFAULT_DETAILS = {"return_logits": True, "return_latents": True, "return_head": False, "return_stats": False}


class RavenPreTrainedModel(PreTrainedModel):
    config_class = RavenConfig
    base_model_prefix = "model"
    supports_gradient_checkpointing = True
    _no_split_modules = ["SandwichBlock"]
    _skip_keys_device_placement = ["past_key_values"]
    _tied_weights_keys = {"lm_head.weight": "transformer.wte.weight"}
    _supports_cache_class = True

    def _init_weights(self, module):
        """Weights are initialised by the block constructors (role-aware truncated normals); nothing to redo."""
        return


class RavenForCausalLM(RavenPreTrainedModel, RavenGenerationMixin, GenerationMixin):
    def __init__(self, config: RavenConfig):
        super().__init__(config)
        self.config = config
        mc = config.to_model_config()
        self.model_config = mc
        E = config.n_embd
        P, R, C = config.n_layers_in_prelude, config.n_layers_in_recurrent_block, config.n_layers_in_coda
        init = mc.init
        off = P + R * config.mean_recurrence
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.padded_vocab_size, E),
            prelude=nn.ModuleList(make_block(mc, i) for i in range(P)),
            adapter=Linear(2 * E, E, bias=config.bias, init=lambda w: init.init_weight_(w, "in_proj", P)),
            core_block=nn.ModuleList(make_block(mc, i + P) for i in range(R)),
            coda=nn.ModuleList(make_block(mc, i + off) for i in range(C)),
            ln_f=make_norm(mc)))
        init.init_weight_(self.transformer.wte.weight, "embedding")
        # The reference's inference model draws the up half of every gated-MLP input projection with the (smaller)
        # output-projection deviation, unlike its training model (recpre/raven_modeling_minimal.py:103-104); a freshly
        # constructed model follows it.  Loaded checkpoints overwrite all of this.
        with torch.no_grad():
            for name, module in self.transformer.named_modules():
                if name.endswith("mlp.fc") and getattr(module, "weight", None) is not None \
                        and not mc.skip_initialization:
                    half = module.weight.shape[0] // 2
                    init.normal_(module.weight[half:], std=float(config.init_values["out_proj"]))
        self.emb_scale = config.init_values["embed_scale"]
        self.lm_head = nn.Linear(E, config.padded_vocab_size, bias=False)
        if config.tie_embeddings:
            self.lm_head.weight = self.transformer.wte.weight
        cos, sin = ref.rope_tables(E // config.n_heads, config.block_size, config.rope_base, 1)
        self.register_buffer("freqs_cis", ref.freqs_cis_buffer(cos, sin), persistent=True)
        self.gradient_checkpointing = False
        self.post_init()

    def _apply(self, fn, recurse=True):
        """The rotary table stays fp32 whatever the model is cast to; device moves still apply."""
        keep = self._buffers.get("freqs_cis")
        out = super()._apply(fn, recurse)
        cur = self._buffers.get("freqs_cis")
        if keep is not None and cur is not None and cur.dtype != torch.float32:
            self._buffers["freqs_cis"] = keep.to(device=cur.device, dtype=torch.float32)
        return out

    # -- HF plumbing ---------------------------------------------------------------------------------
    def get_input_embeddings(self):
        return self.transformer.wte

    def get_output_embeddings(self):
        return self.lm_head

    def tie_weights(self, *a, **k):
        if self.config.tie_embeddings:
            self.lm_head.weight = self.transformer.wte.weight

    # -- pieces --------------------------------------------------------------------------------------
    def _rope(self, seq_len: int, position_ids=None, cache_position=None):
        fc = self.freqs_cis[0, :, 0]
        if position_ids is not None:
            fc = fc.index_select(0, position_ids.reshape(-1))
        elif cache_position is not None:
            fc = fc[cache_position]
        else:
            fc = fc[:seq_len]
        return fc[..., 0].contiguous(), fc[..., 1].contiguous()

    _attn_mask = None      # boolean [B, 1, Sq, Sk] of the forward pass in flight, or None (plain causal attention)
    # The reference's forward builds no mask at all (its call of compile_mask is commented out,
    # recpre/raven_modeling_minimal.py:683), so padded rows of a batch attend to their padding.  False keeps that
    # behaviour (bit-level parity of logits); True applies compile_mask, which is what padded batches need.
    apply_padding_mask = False

    def compile_mask(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                     past_key_values=None, pad_token_id: int = 65509) -> Optional[torch.Tensor]:
        """Attention mask of a (pre)fill over ``input_ids``: causal, keys that hold the padding token are hidden, and an
        optional ``attention_mask`` is applied on top ([B, Sq, Sk] boolean as in the reference, or the usual [B, Sk] key
        mask).  None when there is nothing to hide, and for single-token steps on a cache (as in
        recpre/raven_modeling_minimal.py:593-636, which returns a flex-attention block mask; here a dense boolean
        [B, 1, Sq, Sk] tensor)."""
        B, S = input_ids.shape
        has_pad = bool((input_ids == pad_token_id).any())
        if attention_mask is None and not has_pad:
            return None
        if past_key_values is not None and S == 1:
            return None
        seen = past_key_values.get_seq_length() if past_key_values is not None else 0
        if seen:                       # a chunk with history: keys of earlier chunks are not described by input_ids
            return None
        keep = torch.ones(S, S, dtype=torch.bool, device=input_ids.device).tril()[None, None]
        keep = keep & (input_ids != pad_token_id)[:, None, None, :]
        if attention_mask is not None:
            am = attention_mask.to(torch.bool)
            keep = keep & (am[:, None, None, :] if am.dim() == 2 else am[:, None])
        return keep

    def _attention(self, attn, x, rope, step_idx: int, cache):
        B, S, E = x.shape
        cos, sin = rope
        qkv = attn.Wqkv(x)
        mask = self._attn_mask
        if mask is not None and mask.shape[-2] == S:
            q, k, v = ops.qk_bias_rope(qkv, attn.qk_bias, cos, sin, attn.n_head, attn.n_kv, attn.head_dim)
            if cache is not None:
                k, v = cache.update(k, v, step_idx)
            if k.shape[1] == mask.shape[-1]:
                return attn.proj(ops.masked_attention(q, k, v, mask).reshape(B, S, E))
            y = ops.causal_attention(q, k, v, None, k.shape[1] - q.shape[1])
            return attn.proj(y.reshape(B, S, E))
        if x.is_cuda and x.dtype == torch.bfloat16 and S > 1 and not torch.is_grad_enabled():
            y = self._native_prefill_attention(attn, qkv, cos, sin, step_idx, cache)
            if y is not None:
                return attn.proj(y)
        q, k, v = ops.qk_bias_rope(qkv, attn.qk_bias, cos, sin, attn.n_head, attn.n_kv, attn.head_dim)
        if cache is not None:
            k, v = cache.update(k, v, step_idx)
        y = ops.causal_attention(q, k, v, None, k.shape[1] - q.shape[1])
        return attn.proj(y.reshape(B, S, E))

    def _native_prefill_attention(self, attn, qkv, cos, sin, step_idx: int, cache):
        """First chunk of a sequence on a GPU: fused bias+RoPE kernel on the packed qkv, KV-cache append from views of
        the rotated tensor, native causal attention on the packed tensor.  Returns None when the chunk has history."""
        from ..ops import attention as A
        from ..ops import cuda as K

        H, Hkv, D = attn.n_head, attn.n_kv, attn.head_dim
        if not A.native_prefill_supported(D):
            return None
        if cache is not None:
            # the token counter advances when step 0 is written, so later steps of the same chunk already include it
            seen = cache.get_seq_length(step_idx)
            if seen != (0 if step_idx == 0 else qkv.shape[1]):
                return None
        B, S, _ = qkv.shape
        qkv_r = K.rope_fwd(qkv.contiguous(), attn.qk_bias, cos.float().contiguous(), sin.float().contiguous(), H, Hkv, D)
        if cache is not None:
            wq, wk = H * D, Hkv * D
            cache.update(qkv_r[..., wq:wq + wk].view(B, S, Hkv, D), qkv_r[..., wq + wk:].view(B, S, Hkv, D), step_idx)
        y, _ = A.fwd(qkv_r, H, Hkv, D, D ** -0.5)
        return y

    def _block(self, block, x, rope, step_idx: int, cache):
        name = type(block).__name__
        att = lambda h: self._attention(block.attn, h, rope, step_idx, cache)  # noqa: E731
        if name == "SandwichBlock":
            x = block.norm_2.forward_add(att(block.norm_1(x)), x)
            return block.norm_4.forward_add(block.mlp(block.norm_3(x)), x)
        if name == "TransformerPreNormBlock":
            x = att(block.norm_1(x)) + x
            return block.mlp(block.norm_2(x)) + x
        if name == "TransformerPostNormBlock":
            x = block.norm_1.forward_add(att(x), x)
            return block.norm_2.forward_add(block.mlp(x), x)
        raise NotImplementedError(f"block class {name} is not supported by the inference model")

    def initialize_state(self, input_embeds, scale: float = 1.0):
        """Truncated normal, sigma = init std * scale * embedding scale (recpre/raven_modeling_minimal.py:804-813)."""
        std = self.config.init_values["std"] * scale
        if std <= 0:
            return torch.zeros_like(input_embeds)
        seed = int(torch.randint(0, 2**31 - 1, (1,)))
        return ops.trunc_normal_state(input_embeds, std * self.emb_scale, seed)

    def _maybe_inject_noise(self, x, current_step: int, renorm: bool = True):
        n0 = self.config.test_time_noise
        if not n0 or n0 <= 0:
            return x
        n = n0 * self.config.init_values["std"] * self.emb_scale
        kind = self.config.test_time_noise_type
        if kind == "geom":
            f = n / (current_step + 1)
        elif kind == "sqrt":
            f = n / math.sqrt(current_step + 1)
        elif kind == "line":
            f = max(n, (self.config.mean_recurrence - current_step) / self.config.mean_recurrence)
        elif kind == "chi":
            f = float(2 * torch.rand(1) * n)
        elif kind == "fixed":
            f = n
        else:
            raise ValueError(kind)
        x = x * (1 - f) + torch.randn_like(x) * f
        return self.transformer.core_block[-1].norm_4(x) if renorm else x

    def _maybe_checkpoint_core_block(self, *args):
        """One recurrence, recomputed in backward when ``gradient_checkpointing`` is on (finetuning)."""
        if self.gradient_checkpointing and torch.is_grad_enabled():
            return torch.utils.checkpoint.checkpoint(self.core_block_forward, *args, use_reentrant=False,
                                                     preserve_rng_state=False, determinism_check="none")
        return self.core_block_forward(*args)

    def core_block_forward(self, x, input_embeds, rope, cache, block_idx: int, current_step: int = 0):
        x = self._maybe_inject_noise(x, current_step)
        x = ops.adapter(x, input_embeds.to(x.dtype), self.transformer.adapter.weight)
        for block in self.transformer.core_block:
            block_idx += 1
            x = self._block(block, x, rope, block_idx, cache)
        return x, block_idx

    def randomized_iteration_sampler(self):
        """Log-normal Poisson depths on the global RNG in training mode, (mean_recurrence, 0) in eval mode."""
        t = max(self.config.mean_recurrence - self.config.mean_backprop_depth, 0)
        s = self.config.mean_backprop_depth
        if not self.training:
            return self.config.mean_recurrence, 0
        sigma = 0.5
        mu = math.log(t + s) - sigma**2 / 2
        rate = torch.zeros((1,)).log_normal_(mean=mu, std=sigma)
        p = int(torch.poisson(torch.tensor([float(rate)]))) + 1
        return max(p - s, 0), min(s, p)

    def iterate_forward(self, input_embeds, input_states, rope, block_idx, cache, num_steps=None, init_scale=1.0):
        x = xk = self.initialize_state(input_embeds, init_scale) if input_states is None else input_states.clone()
        if num_steps is None:
            n, k = self.randomized_iteration_sampler()
        elif hasattr(num_steps, "__len__") and len(num_steps) > 1:
            n, k = int(num_steps[0]), int(num_steps[1])
        else:
            n, k = int(num_steps), 0
        with torch.no_grad():
            for step in range(n):
                xk = x
                x, block_idx = self.core_block_forward(x, input_embeds, rope, cache, block_idx, step)
        for step in range(k):
            xk = x
            if self.gradient_checkpointing and self.training:
                x, block_idx = torch.utils.checkpoint.checkpoint(self.core_block_forward, x, input_embeds, rope, cache,
                                                                 block_idx, n + step, use_reentrant=False)
            else:
                x, block_idx = self.core_block_forward(x, input_embeds, rope, cache, block_idx, n + step)
        return self.transformer.ln_f(x), n, k, xk.detach(), block_idx

    # -- forward -------------------------------------------------------------------------------------
    def forward(self, input_ids: Optional[torch.Tensor] = None, input_embeds=None, input_states=None,
                attention_mask=None, position_ids=None, labels=None, num_steps=None, past_key_values=None,
                output_details: dict = _DEFAULT_DETAILS, use_cache: bool = False, cache_position=None,
                init_scale: float = 1.0, **kwargs) -> CausalLMOutputRecurrentLatents:
        S = input_ids.shape[1] if input_ids is not None else input_embeds.shape[1]
        rope = self._rope(S, position_ids, cache_position)
        self._attn_mask = self.compile_mask(input_ids, attention_mask, past_key_values) \
            if (self.apply_padding_mask and input_ids is not None) else None
        try:
            return self._forward(input_ids, input_embeds, input_states, rope, labels, num_steps, past_key_values,
                                 output_details, use_cache, init_scale)
        finally:
            self._attn_mask = None

    def _forward(self, input_ids, input_embeds, input_states, rope, labels, num_steps, past_key_values, output_details,
                 use_cache, init_scale) -> CausalLMOutputRecurrentLatents:
        if input_embeds is None:
            input_embeds = ops.embedding(input_ids, self.transformer.wte.weight, self.emb_scale)
        elif self.emb_scale != 1:
            input_embeds = input_embeds * self.emb_scale
        if use_cache and past_key_values is None:
            past_key_values = RecurrentKVCache(core_layers=self.config.n_layers_in_recurrent_block,
                                               prelude_layers=self.config.n_layers_in_prelude)
        block_idx = -1
        for block in self.transformer.prelude:
            block_idx += 1
            input_embeds = self._block(block, input_embeds, rope, block_idx, past_key_values)
        x, n, k, xk, block_idx = self.iterate_forward(input_embeds, input_states, rope, block_idx, past_key_values,
                                                      num_steps, init_scale)
        latent_states = x.detach().clone()
        head_idx = 0
        for block in self.transformer.coda:
            head_idx -= 1
            x = self._block(block, x, rope, head_idx, past_key_values)
        x = self.transformer.ln_f(x)
        logits = ops.linear(x, self.lm_head.weight).float()
        if labels is not None:
            loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1),
                                                     ignore_index=-100)
            log_ppl = loss.detach().clone()
        else:
            loss, log_ppl = torch.as_tensor(0.0), torch.as_tensor(0.0)
        return CausalLMOutputRecurrentLatents(
            loss=loss, log_ppl=log_ppl, logits=logits if output_details["return_logits"] else None,
            past_key_values=past_key_values, hidden_states=x if output_details["return_head"] else None,
            latent_states=latent_states if output_details["return_latents"] else None,
            stats=self.get_stats(logits, x, latent_states, xk, input_embeds, n, k)
            if output_details["return_stats"] else None)

    # -- alternative entry points (used by the samplers and by external evaluation code) ---------------
    @torch.no_grad()
    def embed_inputs(self, input_ids, attention_mask=None, position_ids=None, past_key_values=None,
                     use_cache: bool = False, cache_position=None, **kwargs):
        rope = self._rope(input_ids.shape[1], position_ids, cache_position)
        e = ops.embedding(input_ids, self.transformer.wte.weight, self.emb_scale)
        if use_cache and past_key_values is None:
            past_key_values = RecurrentKVCache(core_layers=self.config.n_layers_in_recurrent_block,
                                               prelude_layers=self.config.n_layers_in_prelude)
        block_idx = -1
        for block in self.transformer.prelude:
            block_idx += 1
            e = self._block(block, e, rope, block_idx, past_key_values)
        return e, block_idx

    @torch.no_grad()
    def iterate_one_step(self, input_embeds, input_states, position_ids=None, cache_position=None, block_idx=0,
                         attention_mask=None, past_key_values=None, current_step: int = 0):
        rope = self._rope(input_embeds.shape[1], position_ids, cache_position)
        x, block_idx = self.core_block_forward(input_states, input_embeds, rope, past_key_values, int(block_idx),
                                               current_step)
        return x, block_idx, current_step + 1

    def predict_from_latents(self, latents, attention_mask=None, position_ids=None, cache_position=None,
                             past_key_values=None):
        rope = self._rope(latents.shape[1], position_ids, cache_position)
        x = self.transformer.ln_f(latents)
        head_idx = 0
        for block in self.transformer.coda:
            head_idx -= 1
            x = self._block(block, x, rope, head_idx, past_key_values)
        x = self.transformer.ln_f(x)
        logits = ops.linear(x, self.lm_head.weight).float()
        return CausalLMOutputRecurrentLatents(loss=torch.as_tensor(0.0), log_ppl=torch.as_tensor(0.0), logits=logits,
                                              past_key_values=past_key_values, latent_states=x)

    @torch.no_grad()
    def _prefill_with_varied_exit_steps(self, input_ids, exit_evaluator, past_key_values=None, init_scale: float = 1.0):
        """Token-by-token "prefill" in which every position iterates until the exit criterion fires (at most
        ``mean_recurrence`` steps).  Deliberately ignores the parallelism of causal attention: a tool for adaptive
        compute experiments (recpre/raven_modeling_minimal.py:936-997).  Batch size 1."""
        assert input_ids.shape[0] == 1, "per-position adaptive depth is defined for a single sequence"
        if past_key_values is None:
            past_key_values = RecurrentKVCache(core_layers=self.config.n_layers_in_recurrent_block,
                                               prelude_layers=self.config.n_layers_in_prelude)
        rows, compute_steps = [], []
        for pos in range(input_ids.shape[1]):
            where = torch.tensor([pos], device=input_ids.device)
            aux = {"cache_position": where, "past_key_values": past_key_values, "attention_mask": None}
            e, block_idx = self.embed_inputs(input_ids[:, pos:pos + 1], use_cache=True, **aux)
            x = self.initialize_state(e, scale=init_scale)
            exit_evaluator.init(x)
            taken = 0
            for step in range(self.config.mean_recurrence):
                x, block_idx, _ = self.iterate_one_step(e, x, block_idx=block_idx, current_step=step, **aux)
                taken = step + 1
                new_exits, _, _ = exit_evaluator.check(self, x, aux)
                if bool(new_exits.any()):
                    break
            compute_steps.append(taken)
            rows.append(self.predict_from_latents(x, cache_position=where, past_key_values=past_key_values).logits)
        return torch.cat(rows, dim=1), past_key_values, compute_steps

    @torch.no_grad()
    def forward_with_adaptive_compute(self, input_ids, exit_evaluator, labels=None, past_key_values=None,
                                      output_details: dict = _DEFAULT_DETAILS, init_scale: float = 1.0, **kwargs):
        """Forward pass with a per-position recurrence count chosen by ``exit_evaluator``; ``stats["compute_steps"]``
        lists the count per position (recpre/raven_modeling_minimal.py:999-1035)."""
        logits, past_key_values, steps = self._prefill_with_varied_exit_steps(input_ids, exit_evaluator, past_key_values,
                                                                              init_scale)
        if labels is not None:
            loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), labels.reshape(-1))
            log_ppl = loss.detach().clone()
        else:
            loss, log_ppl = torch.as_tensor(0.0), torch.as_tensor(0.0)
        return CausalLMOutputRecurrentLatents(loss=loss, log_ppl=log_ppl,
                                              logits=logits if output_details["return_logits"] else None,
                                              past_key_values=past_key_values, stats={"compute_steps": steps})

    @torch.no_grad()
    def get_stats(self, logits, x, latents, xk, input_embeds, n, k) -> dict:
        probs = torch.softmax(logits.float(), dim=-1)
        return {"entropy": float(-(probs * torch.log(probs + 1e-10)).sum(-1).mean()),
                "residual": float((x.float() - latents.float()).norm(dim=-1).mean()),
                "rel_residual": float(((latents.float() - xk.float()).norm(dim=-1) / latents.float().norm(dim=-1)).mean()),
                "num_steps_no_grad": n, "num_steps_with_grad": k}

    # -- conversion ------------------------------------------------------------------------------------
    @classmethod
    def from_training_model(cls, model, dtype: Optional[torch.dtype] = None) -> "RavenForCausalLM":
        """Build the inference model from a training ``RecurrentGPT`` (same state-dict keys; weights are copied)."""
        hf = cls(RavenConfig.from_model_config(model.config))
        sd = {k: v for k, v in model.state_dict().items()}
        hf.load_state_dict(sd, strict=True)
        if dtype is not None:
            hf = hf.to(dtype)
        return hf
