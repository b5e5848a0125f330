"""Training models: the depth-recurrent LM and the plain GPT baseline.

Forward contract (recpre/model_dynamic.py:1075-1162): ``model(input_ids, position_ids=, labels=,
attention_mask=, return_logits=, num_steps_pair=) -> {"loss", "logits", "log_ppl"}``.  The recurrent
model embeds, runs the prelude, draws a state, iterates the core ``n`` times without a graph and
``k`` times with one (input re-injected each time), then ``ln_f -> coda -> ln_f -> tied head``.
State-dict keys are ``transformer.{wte,prelude.i,adapter,core_block.i,coda.i,ln_f}.*``,
``lm_head.weight`` and the fp32 buffer ``freqs_cis`` of shape [1, S, 1, hd/2, 2].

B200 design notes.  The residual stream is bf16 on the GPU; no activation checkpointing is needed at
micro-batch 1 x 4096 tokens (about 33 GB of saved activations for k = 8 out of 180 GB), so the
``gradient_checkpointing`` flag re-computes only when asked.  The loss uses the fused linear +
cross-entropy op, which never materialises the [tokens, vocab] logits unless ``return_logits``.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.nn as nn
import torch.utils.checkpoint

from ..ops import functional as ops
from ..ops import reference as ref
from ..utils import nvtx
from .blocks import Linear, make_block, make_mlp, make_norm
from .sampler import sample_recurrence

# e We^T (the input half of the linear adapter) is the same in every recurrence: compute it once per forward pass
HOIST_ADAPTER = os.environ.get("B200_HOIST_ADAPTER", "1") == "1"


def _rank() -> int:
    import torch.distributed as dist

    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


class _LMBase(nn.Module):
    # Set by the data-parallel stepper for the micro-batch that ends an accumulation window: ``cb(name)`` is called
    # during backward as soon as the gradient of a phase-boundary tensor exists, i.e. when every layer after that
    # boundary has finished its backward pass and its weight gradients are complete (parallel/p2p.py).
    _phase_cb = None
    # Set by the data-parallel stepper when part of the previous optimizer update still runs beside this forward pass:
    # ``cb(name)`` is called before the first use of the weights of phase ``name`` ("core", "coda") and makes the
    # current stream wait for that part of the update (parallel/p2p.py: on_forward).
    _fwd_cb = None

    def _fwd_point(self, name: str) -> None:
        cb = self._fwd_cb
        if cb is not None:
            cb(name)

    def _phase(self, t: torch.Tensor, name: str) -> torch.Tensor:
        cb = self._phase_cb
        if cb is not None and torch.is_grad_enabled() and t.requires_grad:
            def hook(grad, _cb=cb, _name=name):
                _cb(_name)

            t.register_hook(hook)
        return t

    def _ckpt(self):
        """Checkpoint callable for the configured policy (plain recomputation, or selectively kept GEMM / attention
        outputs: ``sac``, ``sac-attn``, ``sac%N`` in ``activation_checkpoint_impl``)."""
        fn = getattr(self, "_ckpt_fn", None)
        if fn is None:
            from ..ops.sac import checkpoint_fn

            fn = self._ckpt_fn = checkpoint_fn(self.config.activation_checkpoint_impl)
        return fn

    def _apply(self, fn, recurse=True):
        """The rotary table stays fp32 whatever the module is cast to (``.bfloat16()`` would otherwise round cos / sin
        to three digits); device moves still apply."""
        keep = self._buffers.get("freqs_cis")
        out = super()._apply(fn, recurse)
        cur = self._buffers.get("freqs_cis")
        if keep is not None and cur is not None and cur.dtype != torch.float32:
            self._buffers["freqs_cis"] = keep.to(device=cur.device, dtype=torch.float32)
        return out

    def _setup_rope(self, config) -> None:
        length = config.randomize_positions_from or config.block_size
        cos, sin = ref.rope_tables(config.head_size, length, config.rope_settings.rope_base,
                                   config.rope_settings.rope_condense_ratio)
        self.register_buffer("freqs_cis", ref.freqs_cis_buffer(cos, sin), persistent=True)

    def _rope(self, seq_len: int, position_ids: Optional[torch.Tensor]):
        """cos/sin [S, hd/2] fp32 views of the buffer for this call."""
        fc = self.freqs_cis
        if position_ids is None:
            fc = fc[0, :seq_len, 0]
        else:
            fc = fc[0].index_select(0, position_ids.reshape(-1))[:, 0]
        return fc[..., 0].contiguous(), fc[..., 1].contiguous()

    def _loss(self, x, labels, return_logits: bool):
        """Head and loss.  Every value of ``use_fused_head`` takes this one path: the loss is the mean cross entropy
        over ALL labelled positions (ignore value -100) of the scaled logits, plus the optional z-loss.  The
        reference's ``hhe`` head averages per-chunk means over chunks of 1024 rows instead (recpre/utils.py:1629-1668),
        which is the same number only when every chunk carries the same count of labelled positions; its ``cce`` and
        ``full-triton`` heads compute the global mean, as here."""
        cfg = self.config
        scale = cfg.init.logit_scale
        logits = None
        if labels is not None:
            ignore = -100
            if return_logits:
                logits = ops.linear(x, self.lm_head.weight).float() * scale
                loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), labels.view(-1),
                                                         ignore_index=ignore)
                z = self.objective.get("z_regularization", 0.0)
                if z:
                    lse = torch.logsumexp(logits.view(-1, logits.shape[-1]), dim=-1)
                    valid = labels.view(-1) != ignore
                    loss = loss + z * (lse.pow(2) * valid).sum() / valid.sum().clamp(min=1)
            else:
                tele = None
                if getattr(self, "monitoring", False) and x.is_cuda:
                    tele = torch.zeros(4, dtype=torch.float32, device=x.device)
                loss = ops.linear_cross_entropy(x, self.lm_head.weight, labels, scale, ignore,
                                                self.objective.get("z_regularization", 0.0), telemetry=tele)
                if tele is not None:      # head statistics of this step (mean over the positions that carry a label)
                    n = (labels != ignore).sum().clamp(min=1).float()
                    t = (tele / n).tolist()
                    self.head_metrics = {"logit_max": t[0], "logit_entropy": t[1], "logit_norm": t[2], "logit_z": t[3]}
            return loss, logits, loss.detach().clone()
        logits = ops.linear(x, self.lm_head.weight).float() * scale
        zero = torch.zeros((), device=x.device)
        return zero, logits, zero


def _accept_transposed_head(module: nn.Module) -> None:
    """The reference's Triton head keeps ``lm_head.weight`` as [E, V] (untied ``full-triton`` head of the recurrent model,
    every GPT baseline: recpre/ops.py:1084-1088); here the head is always [V, E].  Checkpoints in the other layout are
    transposed while they load."""

    def hook(state_dict, prefix, *_):
        key = prefix + "lm_head.weight"
        w = state_dict.get(key)
        want = module.lm_head.weight.shape
        if w is not None and w.dim() == 2 and tuple(w.shape) != tuple(want) and tuple(w.shape) == tuple(want)[::-1]:
            state_dict[key] = w.t().contiguous()

    module._register_load_state_dict_pre_hook(hook)


class RecurrentGPT(_LMBase):
    def __init__(self, config, objective: Optional[dict] = None, gradient_checkpointing: bool = False, **_):
        super().__init__()
        self.config = config
        self.objective = objective or {"ignore_index": -100, "z_regularization": 0.0}
        E = config.n_embd
        P, R, C = config.n_layers_in_prelude, config.n_layers_in_recurrent_block, config.n_layers_in_coda
        init = config.init
        prelude = nn.ModuleList(make_block(config, i) for i in range(P))
        if config.injection_type == "linear":
            adapter = Linear(2 * E, E, bias=config.bias, init=lambda w: init.init_weight_(w, "in_proj", P))
        elif config.injection_type == "ffn":
            adapter = make_mlp(config, 0, in_features=2 * E)
        else:
            adapter = nn.Identity()
        core = nn.ModuleList(make_block(config, i + P) for i in range(R))
        off = P + R * config.mean_recurrence
        coda = nn.ModuleList(make_block(config, i + off) for i in range(C))
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.padded_vocab_size, E), prelude=prelude, adapter=adapter, core_block=core,
            coda=coda, ln_f=make_norm(config)))
        self.emb_scale = init.embedding_scale
        self.lm_head = Linear(E, config.padded_vocab_size, bias=False,
                              init=lambda w: init.init_weight_(w, "head"))
        if config.tie_embeddings:
            self.lm_head.weight = self.transformer.wte.weight
        _accept_transposed_head(self)
        if getattr(config, "embed_step", False):
            from .variants import TimestepEmbedder

            self.step_embedding = TimestepEmbedder(E)
        self._modulated_core = type(core[0]).__name__ == "ModulatedTransformerPostNormBlock" if R else False
        self.max_seq_length = config.block_size
        self.gradient_checkpointing = gradient_checkpointing
        self._setup_rope(config)
        self.step = 0
        self.monitoring = False
        self.latest_metrics: dict = {}
        self.last_depths = (0, 0)
        init.init_weight_(self.transformer.wte.weight, "embedding")

    # -- pieces ------------------------------------------------------------------------
    def state_sigma(self) -> float:
        return self.config.init.get_std("embedding") * self.emb_scale * self.config.state_init_scale

    def initialize_state(self, e: torch.Tensor) -> torch.Tensor:
        """Random start state (recpre/model_dynamic.py:1353-1372); ``like-init`` is a +-3 sigma truncated
        normal with sigma = sqrt(2/(5E)) * sqrt(E) for the ``takase`` family."""
        mode = self.config.state_init
        if self.config.injection_type == "none":
            return e
        if mode == "like-init":
            seed = (self.step * 7919 + 104729 * (_rank() + 1)) & 0x7FFFFFFF
            if not self.training:
                seed = 12345
            return ops.trunc_normal_state(e, self.state_sigma(), seed)
        if mode == "normal":
            return torch.randn_like(e)
        if mode == "embed":
            return torch.randn_like(e) / math.sqrt(e.shape[-1])
        if mode == "zero":
            return torch.zeros_like(e)
        if mode == "unit":
            x = torch.randn_like(e)
            std, mean = torch.std_mean(x, dim=-1, keepdim=True)
            return (x - mean) / std
        raise ValueError(f"unknown state_init {mode!r}")

    def sample_depths(self) -> tuple[int, int]:
        c = self.config
        return sample_recurrence(c.sampling_scheme, c.mean_recurrence, c.mean_backprop_depth, self.step,
                                 training=self.training, rank=_rank(), lockstep_n=c.lockstep_n,
                                 lockstep_k=c.lockstep_k)

    def randomized_iteration_sampler(self):
        n, k = self.sample_depths()
        return torch.as_tensor(n, dtype=torch.long), torch.as_tensor(k, dtype=torch.long)

    def core_block_forward(self, x, e, rope, mask, step: int, inj=None):
        c = self.config
        inj_e, inj = inj, c.injection_type
        context = None
        if getattr(c, "embed_step", False):
            context = self.step_embedding(torch.as_tensor([step], device=e.device)).to(x.dtype)
        if inj == "modulated":  # pairs with ModulatedTransformerPostNormBlock: the state modulates itself
            context = x.clone()
        elif inj == "add":
            x = x + e
        elif inj == "gate":
            x = x * e
        elif inj == "linear" and inj_e is not None:
            x = ops.adapter_state(x, inj_e, self.transformer.adapter.weight)   # e We^T was hoisted out of the loop
        elif inj == "linear":
            x = ops.adapter(x, e, self.transformer.adapter.weight)
            if self.transformer.adapter.bias is not None:
                x = x + self.transformer.adapter.bias.to(x.dtype)
        elif inj == "ffn":
            x = self.transformer.adapter(torch.cat([x, e], dim=-1))
        elif inj != "none":
            raise ValueError("Invalid injection type")
        noise = c.intermediate_noise_injection
        if noise > 0:
            if c.geom_noise_injection == "geom":
                f = noise / (step + 1)
            elif c.geom_noise_injection == "sqrt":
                f = noise / math.sqrt(step + 1)
            elif c.geom_noise_injection == "line":
                top = max(int(getattr(c, "maximal_recurrence", None) or c.mean_recurrence), 1)
                f = max(noise, (top - step) / top)
            elif c.geom_noise_injection == "chi":
                # as in the reference (recpre/model_dynamic.py:1227-1228): a noise level is drawn and not applied;
                # the draw is kept so that the random stream stays the same
                torch.rand(1, device=x.device, dtype=x.dtype)
                f = None
            else:
                f = noise
            if f is not None:
                x = x * (1 - f) + torch.randn_like(x) * f
        per_block = self.gradient_checkpointing and "per-block" in c.activation_checkpoint_impl
        if self._modulated_core:
            for block in self.transformer.core_block:
                x = block(x, rope, mask, context=context)
            return x
        if context is not None:
            x = x + context
        for block in self.transformer.core_block:
            if per_block and torch.is_grad_enabled():
                x = self._ckpt()(block, x, rope, mask)
            else:
                x = block(x, rope, mask)
        return x

    def iterate_forward(self, e, rope, mask, num_steps_pair=None, input_states=None):
        x = self.initialize_state(e) if input_states is None else input_states
        if num_steps_pair is None:
            n, k = self.sample_depths()
        else:
            pair = [int(v) for v in torch.as_tensor(num_steps_pair).reshape(-1).tolist()]
            n, k = (pair[0], pair[1]) if len(pair) > 1 else (pair[0], 0)
        self.last_depths = (n, k)
        offset = 0
        if getattr(self.config, "randomize_embed_step", False):     # recpre/model_dynamic.py:1175-1178
            offset = int(torch.randint(0, self.config.mean_recurrence * 8, (1,), device=e.device))
        xk = x
        inj = None
        if (HOIST_ADAPTER and self.config.injection_type == "linear" and e.is_cuda and n + k > 1
                and self.transformer.adapter.bias is None and x.dtype == e.dtype):
            inj = ops.adapter_inject(e, self.transformer.adapter.weight)
        with torch.no_grad():
            for step in range(n):
                xk = x
                x = self.core_block_forward(x, e, rope, mask, step + offset, inj)
        per_iter = self.gradient_checkpointing and "per-iteration" in self.config.activation_checkpoint_impl
        for step in range(k):
            xk = x
            if per_iter and torch.is_grad_enabled():
                x = self._ckpt()(self.core_block_forward, x, e, rope, mask, n + step + offset, inj)
            else:
                x = self.core_block_forward(x, e, rope, mask, n + step + offset, inj)
        return self.transformer.ln_f(x), n, k, xk.detach()

    def _hoists_adapter(self) -> bool:
        return (HOIST_ADAPTER and self.config.injection_type == "linear" and self.transformer.adapter.bias is None
                and self.transformer.adapter.weight.is_cuda)

    def contributions_per_step(self, k: int) -> dict:
        """How many gradient contributions each parameter receives in one backward pass with k grad
        iterations: k for the core and the adapter, 2 for a tied embedding/head, 2 for ln_f, else 1."""
        out = {}
        for name, p in self.named_parameters():
            if ".adapter." in name and self._hoists_adapter():
                out[name] = max(k, 0) + (1 if k > 0 else 0)   # k state halves + one hoisted input half
            elif ".core_block." in name or ".adapter." in name:
                out[name] = max(k, 0)
            elif name.endswith("wte.weight") and self.config.tie_embeddings:
                out[name] = 2
            elif ".ln_f." in name:
                out[name] = 2 if k > 0 else 1
            else:
                out[name] = 1
        return out

    # -- forward -----------------------------------------------------------------------
    def forward(self, input_ids, attention_mask=None, position_ids=None, labels=None, return_logits: bool = False,
                num_steps_pair=None, input_states=None):
        cfg = self.config
        S = input_ids.shape[1]
        if cfg.randomize_positions_from is not None and self.training:
            position_ids = torch.sort(torch.randint(0, cfg.randomize_positions_from, (S,),
                                                    device=input_ids.device))[0]
        rope = self._rope(S, position_ids)
        with nvtx.range("prelude"):
            e = ops.embedding(input_ids, self.transformer.wte.weight, self.emb_scale)
            for i, block in enumerate(self.transformer.prelude):
                self._phase(e, f"prelude.{i}")    # gradient of block i's input: blocks i.. have gone backward
                e = block(e, rope, attention_mask)
            self._phase(e, "core")       # gradient of the prelude output: all recurrences and the adapter are done
        with nvtx.range("recurrence"):
            self._fwd_point("core")
            x, n, k, xk = self.iterate_forward(e, rope, attention_mask, num_steps_pair, input_states)
        x_rec = x
        in_coda = self.gradient_checkpointing and "in-coda" in cfg.activation_checkpoint_impl
        with nvtx.range("coda"):
            self._fwd_point("coda")
            for i, block in enumerate(self.transformer.coda):
                self._phase(x, f"coda.{i}")       # gradient of block i's input: coda blocks i.. have gone backward
                if in_coda and torch.is_grad_enabled():
                    x = self._ckpt()(block, x, rope, attention_mask)
                else:
                    x = block(x, rope, attention_mask)
            x = self.transformer.ln_f(x)
        if self.monitoring:
            self.monitor_module(x, x_rec, xk, e, n, k)
        loss, logits, log_ppl = self._loss(x, labels, return_logits or labels is None)
        if labels is not None and self.training:
            if cfg.mcleish_throttle and k > 0:
                loss = loss / k
            if cfg.elbayad_weighing:
                t = cfg.mean_recurrence
                w = torch.arange(1, 16 * t, device=loss.device, dtype=torch.float32) ** cfg.elbayad_exponent
                w = w / torch.sum(torch.arange(1, t + 1, device=loss.device, dtype=torch.float32)
                                  ** cfg.elbayad_exponent)
                loss = loss * (w[n + k] / w[t // 2])
        return {"loss": loss, "logits": logits if (return_logits or labels is None) else None, "log_ppl": log_ppl}

    @torch.no_grad()
    def monitor_module(self, x_out, x_rec, xk, input_embeds, num_steps_no_grad, num_steps_with_grad):
        """Model telemetry for one step, with the reference's metric names and formulas
        (recpre/model_dynamic.py:1374-1405): mean cosine between the centred token vectors of a sequence (minus the
        1/S of the diagonal) for the output and for the recurrent state, their norms, the distance of the state from
        the embedded input and the last recurrence's residual."""
        x_out, x_rec, xk, e = x_out.float(), x_rec.float(), xk.float(), input_embeds.float()
        self.latest_metrics = {
            "last_hidden_token_corr": _token_corr(x_out),
            "recurrent_state_token_corr": _token_corr(x_rec),
            "last_hidden_norm": x_out.norm(dim=-1).mean(),
            "recurrent_state_norm": x_rec.norm(dim=-1).mean(),
            "recurrent_diff": (x_rec - e).norm(dim=-1).mean(),
            "num_steps_no_grad": num_steps_no_grad,
            "num_steps_with_grad": num_steps_with_grad,
            "recurrent_residual": (x_rec - xk).norm(dim=-1).mean(),
            "rel_residual": ((x_rec - xk).norm(dim=-1) / x_rec.norm(dim=-1)).mean(),
        }
        self.latest_metrics.update(getattr(self, "head_metrics", {}))

    def reset_parameters(self) -> None:
        """Re-draw every weight with the config's initialiser (embedding, blocks, adapter, head; norms to one)."""
        _reinitialize(self)


def _token_corr(x: torch.Tensor) -> torch.Tensor:
    c = x - x.mean(dim=-1, keepdim=True)
    c = c / c.norm(dim=-1, keepdim=True)
    return (c @ c.transpose(1, 2)).mean() - 1 / x.shape[1]


def _reinitialize(model: nn.Module) -> None:
    init = model.config.init
    init.init_weight_(model.transformer.wte.weight, "embedding")
    for m in model.modules():
        if m is not model and hasattr(m, "reset_parameters") and not isinstance(m, (RecurrentGPT, GPT)):
            m.reset_parameters()
    init.init_weight_(model.transformer.wte.weight, "embedding")      # nn.Embedding's own reset ran in the loop
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("qk_bias"):
                p.zero_()


class GPT(_LMBase):
    """Non-recurrent decoder (recpre/model_dynamic.py:22-144)."""

    def __init__(self, config, objective: Optional[dict] = None, gradient_checkpointing: bool = False, **_):
        super().__init__()
        self.config = config
        self.objective = objective or {"ignore_index": -100, "z_regularization": 0.0}
        init = config.init
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(config.padded_vocab_size, config.n_embd),
            h=nn.ModuleList(make_block(config, i) for i in range(config.n_layer)),
            ln_f=make_norm(config)))
        if config.use_abacus:
            # the reference creates this positional table for its baseline model and never reads it
            # (recpre/model_dynamic.py:36-40); it exists here so that such checkpoints load key for key
            self.transformer["abacus"] = nn.Embedding(config.block_size, config.n_embd)
        self.lm_head = Linear(config.n_embd, config.padded_vocab_size, bias=config.lm_head_bias,
                              init=lambda w: init.init_weight_(w, "head"))
        _accept_transposed_head(self)
        self.emb_scale = math.sqrt(config.n_embd) if config.scale_embeddings else init.embedding_scale
        self.gradient_checkpointing = gradient_checkpointing
        self.max_seq_length = config.block_size
        self._setup_rope(config)
        self.step = 0
        self.monitoring = False
        self.latest_metrics: dict = {}
        self.last_depths = (0, config.n_layer)
        init.init_weight_(self.transformer.wte.weight, "embedding")

    def contributions_per_step(self, k: int) -> dict:
        return {name: 1 for name, _ in self.named_parameters()}

    def forward(self, input_ids, attention_mask=None, position_ids=None, labels=None, return_logits: bool = False,
                num_steps_pair=None, **_):
        S = input_ids.shape[1]
        rope = self._rope(S, position_ids)
        x = ops.embedding(input_ids, self.transformer.wte.weight, self.emb_scale)
        half = len(self.transformer.h) // 2
        for i, block in enumerate(self.transformer.h):
            if i == half and i > 0:
                self._phase(x, "upper")  # gradient here: the upper half of the stack has gone backward
            if self.gradient_checkpointing and torch.is_grad_enabled():
                x = self._ckpt()(block, x, rope, attention_mask)
            else:
                x = block(x, rope, attention_mask)
        x = self.transformer.ln_f(x)
        if self.monitoring:
            self.monitor_module(x)
        loss, logits, log_ppl = self._loss(x, labels, return_logits or labels is None)
        return {"loss": loss, "logits": logits if (return_logits or labels is None) else None, "log_ppl": log_ppl}

    @torch.no_grad()
    def monitor_module(self, x: torch.Tensor) -> None:
        """Telemetry of the baseline model (recpre/model_dynamic.py:139-144)."""
        x = x.float()
        self.latest_metrics = {"last_hidden_token_corr": _token_corr(x), "last_hidden_norm": x.norm(dim=-1).mean()}
        self.latest_metrics.update(getattr(self, "head_metrics", {}))

    def reset_parameters(self) -> None:
        _reinitialize(self)
