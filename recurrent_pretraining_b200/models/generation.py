"""Generation paths of the inference model.

``generate`` dispatches on its keyword arguments exactly as the reference does
(recpre/raven_modeling_minimal.py:1112-1127): ``criterion | exit_threshold | exit_evaluator`` select adaptive compute,
``draft_steps | lookahead_for_draft | verification_threshold`` self-speculative decoding,
``headway | state_noise_mixing | inner_recurrence | freeze_strategy`` the diffusion-style sampler, ``continuous_compute``
the minimal loop; anything else runs the minimal loop as well (the reference defers to ``transformers.generate`` there,
whose custom-cache flow broke with transformers 5).

Token sampling order: repetition / DRY penalty -> temperature -> softmax -> top-k -> top-p -> min-p -> renormalise ->
multinomial; greedy argmax when ``do_sample`` is false.  Stop ids are {65504, 65505, 65508} plus ``eos_token_id`` plus
the first token of every stop string.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Optional, Union

import torch
import torch.nn.functional as F

from .exit_criteria import get_adaptive_exit_evaluator
from .kv_cache import RecurrentKVCache

DEFAULT_STOPS = (65504, 65505, 65508)  # begin_text, end_text, end_turn


def _gen_config(model, generation_config):
    gc = generation_config if generation_config is not None else getattr(model, "generation_config", None)
    if gc is None:
        gc = SimpleNamespace()
    defaults = dict(max_length=getattr(model.config, "block_size", 4096), do_sample=False, temperature=None, top_k=None,
                    top_p=None, min_p=None, repetition_penalty=None, eos_token_id=None, stop_strings=None,
                    return_dict_in_generate=False)
    for k, v in defaults.items():
        if not hasattr(gc, k):
            setattr(gc, k, v)
    return gc


class GenerateOutput(dict):
    """``return_dict_in_generate`` result: sequences, scores (per-token recurrence counts and criterion values for
    adaptive decoding) and the cache."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e


class RavenGenerationMixin:
    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, *args, **kwargs):
        if any(k in kwargs for k in ("criterion", "exit_threshold", "exit_evaluator")):
            return self.generate_with_adaptive_compute(*args, **kwargs)
        if any(k in kwargs for k in ("draft_steps", "lookahead_for_draft", "verification_threshold")):
            return self.generate_speculative(*args, **kwargs)
        if any(k in kwargs for k in ("headway", "state_noise_mixing", "inner_recurrence", "freeze_strategy")):
            return self.generate_diffusion_style(*args, **kwargs)
        return self.generate_minimal(*args, **kwargs)

    # ------------------------------------------------------------------------------------------------
    def _prep_generate_args(self, input_ids, generation_config, cache_lookup_strategy, model_kwargs):
        gc = _gen_config(self, generation_config)
        overrides = {k: model_kwargs.pop(k) for k in ("return_dict_in_generate", "do_sample", "temperature", "top_k",
                                                       "top_p", "min_p", "repetition_penalty")
                     if k in model_kwargs}
        if overrides:  # sampling / output options given as plain keyword arguments win over the stored config
            import copy

            gc = copy.copy(gc)
            for k, v in overrides.items():
                setattr(gc, k, v)
        if "max_new_tokens" in model_kwargs:
            max_new = model_kwargs.pop("max_new_tokens")
            if "max_length" in model_kwargs:
                max_new = min(max_new, model_kwargs["max_length"] - input_ids.shape[1])
        else:
            total = model_kwargs.get("max_length", getattr(gc, "max_length", None))
            new = getattr(gc, "max_new_tokens", None)
            if new is not None:                       # a generation config that names the number of new tokens
                max_new = new if total is None else min(new, total - input_ids.shape[1])
            elif total is not None:
                max_new = total - input_ids.shape[1]
            else:
                max_new = 20                              # the library's default length budget
        model_kwargs.pop("max_length", None)
        model_kwargs.pop("cache_implementation", None)
        model_kwargs["past_key_values"] = RecurrentKVCache(
            cache_lookup_strategy, core_layers=self.config.n_layers_in_recurrent_block,
            prelude_layers=self.config.n_layers_in_prelude)
        model_kwargs["use_cache"] = True
        model_kwargs["cache_position"] = torch.arange(input_ids.shape[1], device=input_ids.device)
        return model_kwargs, gc, max(int(max_new), 0)

    def prepare_inputs_for_generation(self, input_ids, past_key_values=None, attention_mask=None, inputs_embeds=None,
                                      cache_position=None, cache_lookup_strategy: str = "full", **kwargs):
        inputs = {"cache_position": cache_position}
        if past_key_values is not None:
            inputs["past_key_values"] = past_key_values if kwargs.get("use_cache", True) else None
            input_ids = input_ids[:, cache_position]
        inputs["input_ids"] = input_ids.contiguous()
        if cache_position is None:
            inputs["position_ids"] = torch.arange(input_ids.shape[1], device=input_ids.device)[None, :]
        for k, v in kwargs.items():
            inputs.setdefault(k, v)
        return inputs

    @staticmethod
    def _advance(model_kwargs):
        """After a token was produced: the next forward consumes exactly one new position."""
        model_kwargs["cache_position"] = model_kwargs["cache_position"][-1:] + 1
        return model_kwargs

    def _get_stops(self, gc, tokenizer, model_kwargs):
        stops = set(DEFAULT_STOPS)
        if gc.eos_token_id is not None:
            try:
                stops.update(gc.eos_token_id)
            except TypeError:
                stops.add(gc.eos_token_id)
        if "stopping_criteria" in model_kwargs and tokenizer is None:
            tokenizer = getattr(model_kwargs["stopping_criteria"][0], "tokenizer", None)
        if getattr(gc, "stop_strings", None) and tokenizer:
            for s in gc.stop_strings:
                stops.add(tokenizer(s, add_special_tokens=False)["input_ids"][0])
        return torch.tensor(sorted(stops))

    # ------------------------------------------------------------------------------------------------
    def _sample_next_token(self, logits, input_ids, gc):
        if gc.repetition_penalty is not None and gc.repetition_penalty != 1.0:
            logits = self._apply_repetition_penalty(logits, input_ids, gc)
        if not gc.do_sample:
            return torch.argmax(logits, dim=-1, keepdim=True)
        logits = logits.to(copy=True, dtype=torch.float32)
        if gc.temperature:
            logits = logits / gc.temperature
        probs = F.softmax(logits, dim=-1)
        if gc.top_k:
            kth = torch.topk(probs, gc.top_k, dim=-1)[0][:, -1:]
            probs = torch.where(probs < kth, torch.zeros_like(probs), probs)
        if gc.top_p:
            sp, si = torch.sort(probs, descending=True, dim=-1)
            remove = torch.cumsum(sp, dim=-1) > gc.top_p
            remove[:, 0] = False
            mask = torch.zeros_like(probs, dtype=torch.bool).scatter(1, si, remove)
            probs = torch.where(mask, torch.zeros_like(probs), probs)
        if gc.min_p:
            probs = torch.where(probs < gc.min_p * probs.max(dim=-1, keepdim=True)[0], torch.zeros_like(probs), probs)
        probs = probs / probs.sum(dim=-1, keepdim=True).clamp(min=1e-10)
        return torch.multinomial(probs, num_samples=1)

    def _apply_repetition_penalty(self, original_logits, input_ids, gc, use_candidates: bool = False):
        """Classic repetition penalty on every token already in the sequence, or the DRY penalty (exponential in the
        length of the repeated n-gram a token would extend) when ``dry_multiplier`` > 0."""
        two_d = original_logits.dim() == 2
        if two_d:
            logits = (original_logits.unsqueeze(1) if original_logits.shape[0] == input_ids.shape[0]
                      else original_logits.unsqueeze(0)).to(copy=True, dtype=torch.float32)
        else:
            logits = original_logits.clone()
        B, T, V = logits.shape
        dry = getattr(gc, "dry_multiplier", 0) or 0
        for b in range(B):
            seq = input_ids[b]
            if use_candidates:
                seq = torch.cat([seq, logits[b].argmax(dim=-1)])
            if dry > 0:
                base, allowed = getattr(gc, "dry_base", 1.75), getattr(gc, "dry_allowed_length", 2)
                ctx = seq.tolist()
                n = len(ctx)
                best: dict = {}
                for start in range(max(0, n - 128), n - 1):
                    m = 0
                    while start + m < n and m < 32 and ctx[start + m] == ctx[n - m - 1]:
                        m += 1
                    if m > 0 and start + m < n:
                        tok = ctx[start + m]
                        best[tok] = max(best.get(tok, 0), m + 1)
                for tok, match in best.items():
                    if match >= allowed:
                        logits[b, :, tok] -= dry * base ** (match - allowed)
            else:
                uniq = torch.unique(seq)
                sel = logits[b][:, uniq]
                logits[b][:, uniq] = torch.where(sel < 0, sel * gc.repetition_penalty, sel / gc.repetition_penalty)
        if two_d:
            return logits.squeeze(1) if original_logits.shape[0] == input_ids.shape[0] else logits.squeeze(0)
        return logits

    def _finish(self, input_ids, gc, model_kwargs, streamer, scores=None, hidden_states=None):
        if streamer:
            streamer.end()
        if gc.return_dict_in_generate:
            return GenerateOutput(sequences=input_ids, scores=scores or {}, logits=None, attentions=None,
                                  hidden_states=hidden_states, past_key_values=model_kwargs.get("past_key_values"))
        return input_ids

    def _update_unfinished(self, unfinished, next_token, stops, model_kwargs, input_ids):
        hit = torch.isin(next_token[:, 0], stops.to(next_token.device))
        unfinished = unfinished & ~hit.long()
        if "stopping_criteria" in model_kwargs:
            unfinished = unfinished & ~model_kwargs["stopping_criteria"](input_ids, None)
        return unfinished

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_minimal(self, input_ids, generation_config=None, tokenizer=None, streamer=None,
                         continuous_compute: bool = False, init_scale: float = 1.0, cache_lookup_strategy: str = "full",
                         **model_kwargs):
        """Token-by-token decoding with a fixed recurrence count (``num_steps`` or the config's mean recurrence).
        ``continuous_compute`` seeds each new token's state with the previous token's final latent."""
        model_kwargs, gc, max_new = self._prep_generate_args(input_ids, generation_config, cache_lookup_strategy,
                                                             model_kwargs)
        stops = self._get_stops(gc, tokenizer, model_kwargs)
        unfinished = torch.ones(input_ids.shape[0], dtype=torch.long, device=input_ids.device)
        if continuous_compute:
            e, _ = self.embed_inputs(input_ids)
            model_kwargs["input_states"] = self.initialize_state(e, scale=init_scale)
        for _ in range(max_new):
            inputs = self.prepare_inputs_for_generation(input_ids, **model_kwargs)
            inputs.pop("stopping_criteria", None)
            out = self(**inputs, init_scale=init_scale)
            logits = out.logits[:, -1, :].to(copy=True, dtype=torch.float32)
            next_token = self._sample_next_token(logits, input_ids, gc)
            input_ids = torch.cat([input_ids, next_token], dim=-1)
            if streamer:
                streamer.put(next_token.cpu())
            model_kwargs = self._advance(model_kwargs)
            if continuous_compute:
                model_kwargs["input_states"] = out.latent_states[:, -1:, :]
            unfinished = self._update_unfinished(unfinished, next_token, stops, model_kwargs, input_ids)
            if int(unfinished.max()) == 0:
                break
        return self._finish(input_ids, gc, model_kwargs, streamer)

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_with_adaptive_compute(self, input_ids, generation_config=None, tokenizer=None, streamer=None,
                                       continuous_compute: bool = False, criterion: str = "none",
                                       exit_threshold: Union[str, float, int] = "auto", init_scale: float = 1.0,
                                       cache_lookup_strategy: str = "full", do_not_exit_in_prefill: bool = False,
                                       min_steps: int = 0, check_criterion_every_n_steps: int = 1,
                                       exit_evaluator=None, **model_kwargs):
        """Per-token adaptive depth: iterate the core until the criterion fires for every live sequence (a sequence's
        logits are frozen at its first exit) or ``num_steps`` is reached.  The per-token step counts and criterion
        traces are returned under ``scores`` when a dict is requested."""
        model_kwargs, gc, max_new = self._prep_generate_args(input_ids, generation_config, cache_lookup_strategy,
                                                             model_kwargs)
        max_steps = model_kwargs.pop("num_steps", self.config.mean_recurrence)
        stops = self._get_stops(gc, tokenizer, model_kwargs)
        B, dev = input_ids.shape[0], input_ids.device
        if continuous_compute:
            e, _ = self.embed_inputs(input_ids)
            model_kwargs["input_states"] = self.initialize_state(e, scale=init_scale)
        unfinished = torch.ones(B, dtype=torch.long, device=dev)
        if exit_evaluator is None:
            exit_evaluator = get_adaptive_exit_evaluator(self, criterion, exit_threshold)
        trace = []
        for t in range(max_new):
            inputs = self.prepare_inputs_for_generation(input_ids, **model_kwargs)
            aux = {k: inputs[k] for k in ("cache_position", "past_key_values", "attention_mask") if k in inputs}
            e, block_idx = self.embed_inputs(inputs["input_ids"], **aux)
            latents = self.initialize_state(e, scale=init_scale) if not continuous_compute \
                else model_kwargs["input_states"]
            next_states = latents[:, -1:, :].clone() if continuous_compute else None
            exit_values = [[] for _ in range(B)]
            steps_taken = [0] * B
            exited = torch.zeros(B, dtype=torch.bool, device=dev)
            outputs, next_logits = None, None
            exit_evaluator.init(latents)
            finished_early = False
            for step in range(max_steps):
                latents, block_idx, _ = self.iterate_one_step(e, latents, block_idx=block_idx, **aux, current_step=step)
                if (step < min_steps or (step - min_steps) % check_criterion_every_n_steps != 0
                        or (do_not_exit_in_prefill and t == 0)):
                    continue
                new_exits, outputs, vals = exit_evaluator.check(self, latents, aux)
                live = ~exited & unfinished.bool()
                vals_host = vals.tolist()  # one transfer per check instead of one per sequence
                for i in range(B):
                    if bool(live[i]):
                        exit_values[i].append(vals_host[i])
                new_exits = new_exits & live
                if bool(new_exits.any()):
                    exited = exited | new_exits
                    if outputs is None:
                        outputs = self.predict_from_latents(latents, **aux)
                    logits = outputs.logits[:, -1, :].to(copy=True, dtype=torch.float32)
                    if next_logits is None:
                        next_logits = logits
                    else:
                        next_logits[new_exits] = logits[new_exits]
                    for i in torch.nonzero(new_exits).flatten().tolist():
                        steps_taken[i] = step + 1
                    if continuous_compute:
                        next_states[new_exits] = latents[new_exits, -1:, :]
                if bool((exited | ~unfinished.bool()).all()):
                    finished_early = True
                    break
            if not finished_early:
                if outputs is None:
                    outputs = self.predict_from_latents(latents, **aux)
                final = outputs.logits[:, -1, :].to(copy=True, dtype=torch.float32)
                if next_logits is None:
                    next_logits = final
                    steps_taken = [max_steps] * B
                else:
                    rest = ~exited & unfinished.bool()
                    next_logits[rest] = final[rest]
                    for i in torch.nonzero(rest).flatten().tolist():
                        steps_taken[i] = max_steps
            if continuous_compute:
                still = ~exited & unfinished.bool()
                next_states[still] = latents[still, -1:, :]
                model_kwargs["input_states"] = next_states
            trace.append([steps_taken, exit_values])
            next_token = self._sample_next_token(next_logits, input_ids, gc)
            input_ids = torch.cat([input_ids, next_token], dim=-1)
            if streamer:
                streamer.put(next_token.cpu())
            model_kwargs = self._advance(model_kwargs)
            unfinished = self._update_unfinished(unfinished, next_token, stops, model_kwargs, input_ids)
            if int(unfinished.max()) == 0:
                break
        scores = {}
        if trace:
            steps, vals = zip(*trace)
            scores = {"compute_steps": list(steps), "exit_values": list(vals)}
        return self._finish(input_ids, gc, model_kwargs, streamer, scores)

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_speculative(self, input_ids, generation_config=None, tokenizer=None, streamer=None,
                             continuous_compute: bool = False, init_scale: float = 1.0,
                             cache_lookup_strategy: str = "full", draft_steps: int = 32, lookahead_for_draft: int = 8,
                             verification_threshold: float = 1, num_steps: int = 32, **model_kwargs):
        """Self-speculative decoding: draft ``lookahead_for_draft`` tokens with ``draft_steps`` recurrences each,
        drop their cache entries, verify all of them in one forward with ``num_steps`` recurrences, keep the agreeing
        prefix plus one corrected token (recpre/raven_modeling_minimal.py:1750-1927).  For batches the shortest
        accepted prefix is applied to every sequence, so no padding is needed and every kept token is verified."""
        assert lookahead_for_draft > 0
        L = lookahead_for_draft
        model_kwargs, gc, max_new = self._prep_generate_args(input_ids, generation_config, cache_lookup_strategy,
                                                             model_kwargs)
        cache = model_kwargs["past_key_values"]
        stops = self._get_stops(gc, tokenizer, model_kwargs)
        unfinished = torch.ones(input_ids.shape[0], dtype=torch.long, device=input_ids.device)
        prefix_len = input_ids.shape[1]
        generated, accepted_log = 0, []

        def run(ids, steps):
            inputs = self.prepare_inputs_for_generation(ids, **model_kwargs)
            inputs.pop("stopping_criteria", None)
            return self(**inputs, num_steps=steps, init_scale=init_scale)

        out = run(input_ids, num_steps)  # prefill at full depth
        tok = self._sample_next_token(out.logits[:, -1, :].float(), input_ids, gc)
        input_ids = torch.cat([input_ids, tok], dim=-1)
        generated += 1
        if streamer:
            streamer.put(tok.cpu())
        unfinished = self._update_unfinished(unfinished, tok, stops, model_kwargs, input_ids)
        model_kwargs["cache_position"] = torch.as_tensor([cache.get_seq_length()], device=input_ids.device)
        if continuous_compute:
            model_kwargs["input_states"] = out.latent_states[:, -1:, :]
        while generated < max_new and int(unfinished.max()) > 0:
            cur = input_ids.shape[1]
            draft = input_ids.clone()
            for _ in range(L):
                out = run(draft, draft_steps)
                tok = self._sample_next_token(out.logits[:, -1, :].float(), draft, gc)
                draft = torch.cat([draft, tok], dim=-1)
                model_kwargs = self._advance(model_kwargs)
                if continuous_compute:
                    model_kwargs["input_states"] = out.latent_states[:, -1:, :]
            cache.clear_last_k_entries(L)
            model_kwargs["cache_position"] = torch.arange(cur - 1, cur + L - 1, device=input_ids.device)
            if continuous_compute:
                model_kwargs.pop("input_states", None)  # the verification pass starts from fresh states
            out = run(draft, num_steps)
            logits = out.logits[:, -L:, :].float()
            drafted = draft[:, cur:]
            if verification_threshold >= 1:
                ok = logits.argmax(dim=-1) == drafted
            else:
                probs = F.softmax(logits, dim=-1)
                ok = probs.gather(-1, drafted.unsqueeze(-1)).squeeze(-1) >= verification_threshold * probs.max(-1)[0]
            bad = ~ok
            first_bad = torch.where(bad.any(dim=1), bad.float().argmax(dim=1), torch.full_like(bad[:, 0], L, dtype=torch.long))
            a = int(first_bad.min())
            pieces = [drafted[:, :a]]
            if a < L:
                corrected = self._sample_next_token(logits[:, a, :], input_ids, gc)
                keep = (first_bad > a).unsqueeze(-1)  # sequences that agreed at position a keep their draft
                pieces.append(torch.where(keep, drafted[:, a:a + 1], corrected))
                cache.clear_last_k_entries(L - a - 1)
            new_tokens = torch.cat(pieces, dim=-1)
            input_ids = torch.cat([input_ids, new_tokens], dim=-1)
            accepted_log.append(new_tokens.shape[1])
            generated += new_tokens.shape[1]
            if streamer:
                streamer.put(new_tokens[0:1].cpu())
            model_kwargs["cache_position"] = torch.as_tensor([cache.get_seq_length()], device=input_ids.device)
            if cache.get_seq_length() < input_ids.shape[1] - 1:  # all drafts accepted: one unprocessed token remains
                model_kwargs["cache_position"] = torch.arange(cache.get_seq_length(), input_ids.shape[1],
                                                              device=input_ids.device)
            if continuous_compute:
                model_kwargs["input_states"] = out.latent_states[:, a:a + 1, :] if a < L else out.latent_states[:, -1:, :]
            hit = torch.isin(new_tokens, stops.to(new_tokens.device)).any(dim=1)
            unfinished = unfinished & ~hit.long()
            if "stopping_criteria" in model_kwargs:
                unfinished = unfinished & ~model_kwargs["stopping_criteria"](input_ids, None)
        # cut every sequence after its first stop token
        pad_id = 65509
        for i in range(input_ids.shape[0]):
            pos = torch.isin(input_ids[i, prefix_len:], stops.to(input_ids.device)).nonzero()
            if len(pos) > 0:
                input_ids[i, prefix_len + int(pos[0]) + 1:] = pad_id
        real = (input_ids != pad_id).any(dim=0).nonzero()
        if len(real) > 0:
            input_ids = input_ids[:, : int(real[-1]) + 1]
        return self._finish(input_ids, gc, model_kwargs, streamer, {"accepted_tokens": accepted_log})

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_diffusion_style(self, input_ids, generation_config=None, tokenizer=None, streamer=None,
                                 init_scale: float = 1.0, cache_lookup_strategy: str = "latest-m4-compress-s4",
                                 full_prefill: bool = True, ema_embeds: float = 0.1, state_noise_mixing: float = 0.5,
                                 inner_recurrence: int = 4, num_steps: int = 32, freeze_strategy: str = "latent-diff",
                                 headway: int = 1, dampened_state_mixer: bool = True, sqrt_mixer: bool = False,
                                 continuous_compute: bool = False, exit_t: float = 0.03, max_wavefront: int = 128,
                                 max_diffusion_steps: int = 4096, return_analysis_tablets: bool = False,
                                 return_full_state_tablet: bool = False, **model_kwargs):
        """Diffusion-style sampling (batch 1): a wavefront of not-yet-frozen positions is refined together, each sweep
        running ``inner_recurrence`` core iterations over the whole front, proposing tokens for every position and
        extending the front by ``headway`` positions; positions freeze (left to right) once their latent stops moving
        (``latent-diff`` < ``exit_t``) or their token has been stable for ``num_steps / inner_recurrence`` sweeps
        (``token-stability``).  Equivalent to ordinary decoding for ``headway = 1, inner_recurrence = num_steps``
        (recpre/raven_modeling_minimal.py:1234-1549).  Freeze strategies: ``latent-diff`` (relative change of the
        latent), ``latent-acceleration-1`` / ``-2`` (relative second difference over the last two / three sweeps),
        ``token-stability``, ``fixed``.  ``return_analysis_tablets`` records, per sweep and on the CPU, the proposed and
        frozen tokens, the recurrence and stability counters (and with ``return_full_state_tablet`` the bf16 latents)
        and returns them as ``hidden_states`` of the output."""
        assert input_ids.shape[0] == 1, "Only batch_size=1 supported"
        model_kwargs, gc, max_new = self._prep_generate_args(input_ids, generation_config, cache_lookup_strategy,
                                                             model_kwargs)
        cache = model_kwargs["past_key_values"]
        stops = self._get_stops(gc, tokenizer, model_kwargs).to(input_ids.device)
        dev, E = input_ids.device, self.config.n_embd
        prompt_len = input_ids.shape[1]
        size = max(self.config.block_size, prompt_len + max_new + headway + 1)
        rec_count = torch.zeros(1, size, dtype=torch.long, device=dev)
        stable = torch.zeros(1, size, dtype=torch.long, device=dev)
        like = self.transformer.wte.weight.new_zeros(1, 1, E) if self.transformer.wte.weight.dtype != torch.float32 \
            else torch.zeros(1, 1, E, device=dev)
        stats = {"core_passes": 0, "tokens_forward": 0, "cache_clears": 0, "standing_waves": 0}
        tablets = None
        if return_analysis_tablets:
            rows = (max_new + headway) * 2
            tablets = {name: torch.zeros(rows, size, dtype=torch.long) for name in ("token_tablet", "frozen_tablet",
                                                                                    "counter_tablet", "stability_tablet")}
            tablets["state_tablet"] = torch.zeros(rows, size, E, dtype=torch.bfloat16) if return_full_state_tablet \
                else None
        if full_prefill:
            inputs = self.prepare_inputs_for_generation(input_ids, **model_kwargs)
            out = self(**inputs, init_scale=init_scale, num_steps=num_steps)
            tok = self._sample_next_token(out.logits[:, -1, :].float(), input_ids, gc)
            frozen = current = torch.cat([input_ids, tok], dim=-1)
            rec_count[:, : frozen.shape[1]] += num_steps
            states = self.initialize_state(out.latent_states[:, -1:, :], scale=init_scale)
        else:
            frozen = current = input_ids.clone()
            states = self.initialize_state(like.expand(1, prompt_len, E), scale=init_scale)
            if 0 < max_wavefront < states.shape[1]:
                raise ValueError("prompt longer than max_wavefront; use full_prefill or raise max_wavefront")
        old_embeds = self.embed_inputs(current)[0] if ema_embeds > 0 else None
        prev_states, old_index, sweeps = states.clone(), 0, 0
        prev_delta, prev_prev_states, old_old_index = torch.zeros_like(states).float(), torch.zeros_like(states), 0
        while frozen.shape[1] - prompt_len < max_new and current.shape[1] <= self.config.block_size \
                and sweeps < max_diffusion_steps:
            sweeps += 1
            idx = cache.get_seq_length()
            n = states.shape[1]
            pos = torch.arange(idx, idx + n, device=dev)
            aux = dict(past_key_values=cache, cache_position=pos)
            e, block_idx = self.embed_inputs(current[:, pos], **aux)
            if ema_embeds > 0:
                old = old_embeds[:, idx - old_index:]
                mixed = e * (1 - ema_embeds)
                mixed[:, : old.shape[1]] += old[:, : mixed.shape[1]] * ema_embeds
                mixed[:, old.shape[1]:] += e[:, old.shape[1]:] * ema_embeds
                e = old_embeds = mixed
            if state_noise_mixing > 0:
                rnd = self.initialize_state(states, scale=init_scale)
                noise = (state_noise_mixing / (1 + rec_count[:, idx: idx + n]))[:, :, None].to(states.dtype) \
                    if dampened_state_mixer else torch.as_tensor(state_noise_mixing, device=dev, dtype=states.dtype)
                states = states * F.relu(1 - noise).sqrt() + noise.sqrt() * rnd if sqrt_mixer \
                    else states * (1 - noise) + noise * rnd
            for _ in range(inner_recurrence):
                states, block_idx, _ = self.iterate_one_step(e, states, block_idx=block_idx, **aux)
                rec_count[:, idx: idx + n] += 1
                stats["core_passes"] += 1
                stats["tokens_forward"] += n
            logits = self.predict_from_latents(states, **aux).logits[0, max(frozen.shape[1] - 1 - idx, 0):, :].float()
            new_tokens = self._sample_next_token(logits, frozen, gc).T
            proposal = torch.cat([frozen, new_tokens[:, :-1]], dim=1)
            stable[:, : current.shape[1]] += (current == proposal[:, : current.shape[1]]).long()
            extra = torch.randint(0, self.config.vocab_size - 26, (1, headway - 1), device=dev)
            current = torch.cat([frozen, new_tokens, extra], dim=1)
            new_state = states[:, -headway:].clone() if continuous_compute and n >= headway else \
                self.initialize_state(like.expand(1, headway, E).to(states.dtype), scale=init_scale)
            states = torch.cat([states, new_state], dim=1)
            head = headway
            if 0 < max_wavefront < states.shape[1]:
                head = max_wavefront - (states.shape[1] - headway)
                states = states[:, :max_wavefront]
                current = current[:, : idx + max_wavefront]
                stats["standing_waves"] += 1
            k = None
            if "latent" in freeze_strategy:
                match_prev = prev_states[:, idx - old_index:]
                cur = states[:, : match_prev.shape[1]]
                match_prev = match_prev[:, : cur.shape[1]]
                first = idx                                   # absolute position of the criterion's first entry
                if freeze_strategy == "latent-diff":
                    crit = (cur - match_prev).float().norm(dim=-1) / cur.float().norm(dim=-1)
                elif freeze_strategy == "latent-acceleration-1":
                    delta = (cur - match_prev).float()
                    m = min(delta.shape[1], prev_delta.shape[1])
                    crit = (delta[:, :m] - prev_delta[:, :m]).norm(dim=-1) / cur[:, :m].float().norm(dim=-1)
                    prev_delta = delta.clone()
                elif freeze_strategy == "latent-acceleration-2":
                    first = max(idx, old_index, old_old_index)
                    last = min(idx + states.shape[1], old_index + prev_states.shape[1],
                               old_old_index + prev_prev_states.shape[1])
                    a = states[:, first - idx: last - idx].float()
                    b = prev_states[:, first - old_index: last - old_index].float()
                    c = prev_prev_states[:, first - old_old_index: last - old_old_index].float()
                    crit = ((a - b) - (b - c)).norm(dim=-1) / (a.norm(dim=-1) + 1e-6)
                else:
                    raise ValueError(f"unknown freeze_strategy {freeze_strategy!r}")
                done = (crit < exit_t).nonzero()
                if len(done) > 0:
                    k = first + int(done[-1][1]) + 1
            elif freeze_strategy == "token-stability":
                done = (stable > num_steps // inner_recurrence).nonzero()
                if len(done) > 0:
                    k = int(done[-1][1]) + 1
            elif freeze_strategy == "fixed":
                done = (rec_count[:, : current.shape[1]] >= num_steps).nonzero()
                if len(done) > 0:
                    k = int(done[-1][1]) + 1
            else:
                raise ValueError(f"unknown freeze_strategy {freeze_strategy!r}")
            prev_prev_states, old_old_index = prev_states, old_index
            prev_states, old_index = states.clone(), idx
            if tablets is not None and sweeps - 1 < tablets["token_tablet"].shape[0]:
                row = sweeps - 1
                tablets["token_tablet"][row, : current.shape[1]] = current[0].cpu()
                tablets["frozen_tablet"][row, : frozen.shape[1]] = frozen[0].cpu()
                tablets["counter_tablet"][row] = rec_count[0].cpu()
                tablets["stability_tablet"][row] = stable[0].cpu()
                if tablets["state_tablet"] is not None:
                    width = min(states.shape[1], size - idx)
                    tablets["state_tablet"][row, idx: idx + width] = states[0, :width].to(torch.bfloat16).cpu()
            if k is not None and k > frozen.shape[1] - 1 and k > idx:
                k = min(k, current.shape[1] - head)
                clear = current.shape[1] - head - k + 1
                cache.clear_last_k_entries(max(min(clear, cache.get_seq_length() - idx), 0))
                stats["cache_clears"] += max(clear, 0)
                new_idx = cache.get_seq_length()
                states = states[:, new_idx - idx:]
                prev_states, old_index = prev_states[:, new_idx - idx:], new_idx
                if streamer:
                    streamer.put(current[:, frozen.shape[1]: k].cpu())
                frozen = current[:, :k]
            else:
                cleared = cache.get_seq_length() - idx
                cache.clear_last_k_entries(cleared)
                stats["cache_clears"] += cleared
            hits = torch.isin(frozen[0, prompt_len:], stops).nonzero()
            if len(hits) > 0:
                frozen = frozen[:, : prompt_len + int(hits[0]) + 1]
                break
        out_ids = frozen[:, : prompt_len + max_new]
        # the reference's names for the same counters (recpre/raven_modeling_minimal.py:1528-1538)
        stats.update(num_core_forward_passes=stats["core_passes"], num_tokens_forward=stats["tokens_forward"],
                     num_cache_clears=stats["cache_clears"], num_standing_waves=stats["standing_waves"],
                     diffusion_steps=sweeps, gen_seq_length=current.shape[1], len_prefill=prompt_len,
                     recurrence_per_position=rec_count[:, : frozen.shape[1]].cpu(),
                     token_stable_per_position=stable[:, : frozen.shape[1]].cpu())
        analysis = None
        if tablets is not None:
            analysis = dict(last_step=sweeps, last_recurrence=sweeps * inner_recurrence, longest_token=current.shape[1],
                            **tablets)
        return self._finish(out_ids, gc, model_kwargs, streamer, stats, hidden_states=analysis)
