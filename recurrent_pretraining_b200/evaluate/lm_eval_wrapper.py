"""Scoring interface in the shape lm-eval expects (``loglikelihood``, ``loglikelihood_rolling``, ``generate_until``)
around a training checkpoint or an HF-style model, at a chosen recurrence.

Counterpart of evaluate_raven/quick_checkpoint_eval.py:50-311.  lm-eval itself is not installed here, so the class
stands alone (its methods take the same request tuples) and registers as an lm-eval ``TemplateLM`` only when the
package can be imported.
"""
from __future__ import annotations

import os

from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

try:  # optional dependency
    from lm_eval.api.model import TemplateLM as _Base  # type: ignore
except Exception:  # pragma: no cover - lm-eval absent
    _Base = object


class RecurrentLM(_Base):
    def __init__(self, model, tokenizer, device=None, batch_size: int = 8, recurrence: Optional[int] = None,
                 max_length: Optional[int] = None, max_gen_toks: int = 512):
        if _Base is not object:
            super().__init__()
        self.model = model.eval()
        self.tokenizer = tokenizer
        self.device = device or next(model.parameters()).device
        self.batch_size = batch_size
        self.recurrence = recurrence or model.config.mean_recurrence
        self.max_length = max_length or model.config.block_size
        self.max_gen_toks = max_gen_toks
        self._hf = hasattr(model, "predict_from_latents")

    @classmethod
    def from_checkpoint(cls, ckpt_path: str, tokenizer, device="cpu", **kw):
        """A raw training checkpoint (this framework's or the reference's) plus a tokenizer object or the folder of a
        Hugging Face tokenizer (evaluate_raven/quick_checkpoint_eval.py:53-79)."""
        from .convert_to_hf import load_training_checkpoint

        if isinstance(tokenizer, (str, os.PathLike)):
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(str(tokenizer))

        cfg, sd = load_training_checkpoint(ckpt_path)
        model = cfg.construct_model()
        model.load_state_dict(sd, strict=False)
        return cls(model.to(device), tokenizer, device=device, **kw)

    # -- tokenizer plumbing ---------------------------------------------------------------------------
    @property
    def eot_token_id(self) -> int:
        return getattr(self.tokenizer, "eos_token_id", None) or getattr(self.tokenizer, "eos_id", 0)

    def tok_encode(self, string: str, **kwargs) -> List[int]:
        try:
            return list(self.tokenizer.encode(string, add_special_tokens=False))
        except TypeError:
            out = self.tokenizer.encode(string)
            return out.tolist() if hasattr(out, "tolist") else list(out)

    def tok_decode(self, tokens, skip_special_tokens: bool = True) -> str:
        return self.tokenizer.decode(list(tokens))

    # -- model plumbing -------------------------------------------------------------------------------
    @torch.no_grad()
    def _logits(self, ids: torch.Tensor) -> torch.Tensor:
        if self._hf:
            return self.model(ids, num_steps=self.recurrence).logits.float()
        out = self.model(ids, num_steps_pair=torch.tensor([self.recurrence, 0]), return_logits=True)
        return out["logits"].float()

    def _loglikelihood_tokens(self, requests: List[Tuple[Tuple[str, str], List[int], List[int]]],
                              disable_tqdm: bool = True, override_bs: Optional[int] = None) -> List[Tuple[float, bool]]:
        """(sum of continuation log-probs, whether the continuation is the greedy decode) per request.  Requests are
        sorted by length and batched with right padding (causal attention makes the padding harmless)."""
        bs = override_bs or self.batch_size
        order = sorted(range(len(requests)), key=lambda i: -(len(requests[i][1]) + len(requests[i][2])))
        results: List[Optional[Tuple[float, bool]]] = [None] * len(requests)
        for b in range(0, len(order), bs):
            idx = order[b:b + bs]
            rows, spans = [], []
            for i in idx:
                _, ctx, cont = requests[i]
                toks = (list(ctx) + list(cont))[-(self.max_length + 1):][:-1]
                rows.append(toks)
                spans.append((len(toks) - len(cont), len(toks)))
            L = max(len(r) for r in rows)
            ids = torch.full((len(rows), L), self.eot_token_id, dtype=torch.long)
            for j, r in enumerate(rows):
                ids[j, :len(r)] = torch.tensor(r)
            logp = F.log_softmax(self._logits(ids.to(self.device)), dim=-1).cpu()
            for j, i in enumerate(idx):
                cont = torch.tensor(requests[i][2][-(spans[j][1] - max(spans[j][0], 0)):])
                lo, hi = max(spans[j][0], 0), spans[j][1]
                sl = logp[j, lo:hi]
                greedy = bool((sl.argmax(-1) == cont).all())
                results[i] = (float(sl.gather(-1, cont[:, None]).sum()), greedy)
        return results  # type: ignore[return-value]

    def loglikelihood(self, requests) -> List[Tuple[float, bool]]:
        reqs = []
        for r in requests:
            ctx, cont = r.args if hasattr(r, "args") else r
            ctx_ids = self.tok_encode(ctx) if ctx else [self.eot_token_id]
            reqs.append(((ctx, cont), ctx_ids, self.tok_encode(cont)))
        return self._loglikelihood_tokens(reqs)

    def loglikelihood_rolling(self, requests, disable_tqdm: bool = True) -> List[float]:
        """Full-document log-likelihood in non-overlapping windows of ``max_length`` tokens, each window conditioned
        on one token of left context."""
        out = []
        for r in requests:
            args = r.args if hasattr(r, "args") else r
            text = args[0] if isinstance(args, (tuple, list)) else args
            toks = [self.eot_token_id] + self.tok_encode(text)
            total = 0.0
            for s in range(0, len(toks) - 1, self.max_length):
                window = toks[s:s + self.max_length + 1]
                total += self._loglikelihood_tokens([(("", ""), window[:1], window[1:])])[0][0]
            out.append(total)
        return out

    @torch.no_grad()
    def generate_until(self, requests, disable_tqdm: bool = True) -> List[str]:
        res = []
        for r in requests:
            ctx, gen_kwargs = r.args if hasattr(r, "args") else r
            until = gen_kwargs.get("until", []) if isinstance(gen_kwargs, dict) else []
            until = [until] if isinstance(until, str) else list(until)
            max_new = int(gen_kwargs.get("max_gen_toks", self.max_gen_toks)) if isinstance(gen_kwargs, dict) else \
                self.max_gen_toks
            ids = torch.tensor([self.tok_encode(ctx)[-(self.max_length - max_new):]], device=self.device)
            text = ""
            for _ in range(max_new):
                nxt = self._logits(ids)[:, -1].argmax(-1, keepdim=True)
                ids = torch.cat([ids, nxt], dim=1)
                if int(nxt) == self.eot_token_id:
                    break
                text += self.tok_decode([int(nxt)])
                if any(u and u in text for u in until):
                    break
            for u in until:
                if u and u in text:
                    text = text.split(u)[0]
            res.append(text)
        return res
