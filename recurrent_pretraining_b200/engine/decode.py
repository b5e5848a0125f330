"""Native decode engine for the depth-recurrent model (the serving hot path; replaces the reference's vLLM plugin,
vllm/raven_vllm.py:297-411, and its HF token loops).

Design for B200:
* weights are streamed once per recurrence by skinny tcgen05 GEMMs computed as ``W x^T`` (weight rows fill the 128-row
  MMA dimension, K is split when ``N/128`` tiles cannot occupy all SMs), so decoding runs at HBM speed;
* the KV cache is a static ``[slots, B, Lmax, H_kv, D]`` tensor pair with one slot per (prelude block | recurrence step
  x core block | coda block) -- the per-recurrence-step cache of the reference -- optionally folded onto fewer slots
  (``compress-s{N}``); q/k bias + RoPE + cache append is one kernel, attention over the cache a split-K
  flash-decoding kernel with per-sequence lengths;
* a whole token (prelude, r recurrences, coda, head, argmax, position bump) is ONE CUDA graph replay for fixed depth;
  with the KL exit each recurrence is a graph, the criterion (log-softmax, KL against the previous step, threshold,
  first-exit bookkeeping) runs in one kernel on the device, and the host looks at a single live-sequence counter
  every ``check_every`` steps;
* ``continuous_compute`` carries each sequence's latent state at its exit step into the next token.

Batch semantics follow the reference's adaptive sampler: all sequences keep iterating until every live sequence has
exited; a sequence's token is frozen at its first exit (recpre/raven_modeling_minimal.py:1646-1693).
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from ..ops import cuda as K

BF16 = torch.bfloat16
_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
_set_pdl = K._sig("b200_set_pdl", [_i])
PDL = os.environ.get("B200_DECODE_PDL", "0") == "1"  # measured within noise of off (23.1-23.5 vs 23.5 ms per token): off
_skinny = K._sig("b200_gemm_skinny", [_vp] * 4 + [_i] * 7 + [_vp, _vp])
_cast_zero = K._sig("b200_cast_zero", [_vp, _vp, C.c_longlong, _vp])
_swiglu_acc = K._sig("b200_swiglu_acc", [_vp, _vp, C.c_longlong, _i, _vp])
_norm_pair = K._sig("b200_add_rmsnorm_pair", [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp])
_rope_append = K._sig("b200_rope_append", [_vp] * 8 + [_i] * 5 + [_vp, _i])
_decode_attn = K._sig("b200_decode_attention", [_vp] * 7 + [_i] * 6 + [_f, _vp])
_kl_exit = K._sig("b200_kl_exit", [_vp] * 7 + [_i, _i, _f, _i, _i, _vp])


class StaticRecurrentKVCache:
    """Static per-step cache with the ``update`` interface of ``RecurrentKVCache`` (used for the prefill through the
    ordinary model forward) and raw slot access for the decode kernels."""

    def __init__(self, n_slots: int, batch: int, max_len: int, n_kv: int, head_dim: int, device, prelude: int, core: int,
                 coda: int, compress: int = 0):
        self.P, self.R, self.Cn, self.compress = prelude, core, coda, compress
        self.n_slots, self.max_len = n_slots, max_len
        self.k = torch.zeros(n_slots, batch, max_len, n_kv, head_dim, dtype=BF16, device=device)
        self.v = torch.zeros_like(self.k)
        self._seen_tokens = 0

    def slot(self, step_idx: int) -> int:
        """Prelude 0..P-1, recurrence steps P.., coda (negative indices) in the last slots."""
        if step_idx < 0:
            return self.n_slots + step_idx
        if step_idx >= self.P and self.compress:
            return (step_idx - self.P) % self.compress + self.P
        return step_idx

    def update(self, k, v, step_idx, lookup_strategy=None):
        step_idx = int(step_idx)
        s = self.slot(step_idx)
        n = k.shape[1]
        if step_idx == 0:
            self._seen_tokens += n
        end = self._seen_tokens
        self.k[s, :, end - n:end] = k
        self.v[s, :, end - n:end] = v
        if end == n:  # first chunk: attend to the fresh (densely packed) tensors, not to strided cache views
            return k, v
        return self.k[s, :, :end], self.v[s, :, :end]

    def get_seq_length(self, step_idx: int = 0) -> int:
        return self._seen_tokens

    def get_memory_usage(self) -> float:
        return 2 * self.k.numel() * 2 / 2**20


class DecodeEngine:
    def __init__(self, model, max_batch: int, max_len: int, num_steps: int | None = None,
                 cache_lookup_strategy: str = "full", use_graphs: bool = True, attn_splits: int = 0,
                 max_steps: int | None = None):
        cfg = model.config
        self.model, self.cfg = model, cfg
        self.dev = next(model.parameters()).device
        assert self.dev.type == "cuda" and next(model.parameters()).dtype == BF16, "engine runs bf16 weights on a GPU"
        assert max_batch <= 64, "decode kernels cover batches up to 64 per replica"
        self.B, self.Lmax = max_batch, max_len
        self.r = num_steps or cfg.mean_recurrence
        self.P, self.R, self.Cn = cfg.n_layers_in_prelude, cfg.n_layers_in_recurrent_block, cfg.n_layers_in_coda
        self.H, self.Hkv, self.D, self.E = cfg.n_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.n_embd
        self.V = cfg.padded_vocab_size
        compress = 0
        if "compress-s" in cache_lookup_strategy:
            compress = int(cache_lookup_strategy.split("compress-s")[1].split("-")[0])
        self.max_steps = max(self.r, max_steps or self.r)  # cache slots exist for this many recurrences
        rec_slots = compress if compress else self.R * self.max_steps
        self.cache = StaticRecurrentKVCache(self.P + rec_slots + self.Cn, max_batch, max_len, self.Hkv, self.D,
                                            self.dev, self.P, self.R, self.Cn, compress)
        self.use_graphs = use_graphs
        # flash-decoding splits of the key range: enough CTAs (128 threads each) to fill every SM's thread slots at small
        # batch -- the per-key walk is latency-bound, so more, shorter walks win (B=1: 16 splits, B=8: 5, B>=32: 1)
        self.splits = attn_splits or max(1, min(16, (16 * 148) // max(1, max_batch * self.H)))
        cos, sin = model._rope(max_len)
        self.cos, self.sin = cos.float().contiguous(), sin.float().contiguous()
        d = self.dev
        self.pos = torch.zeros(max_batch, dtype=torch.int32, device=d)
        self.lens = torch.zeros(max_batch, dtype=torch.int32, device=d)
        self.tok = torch.zeros(max_batch, dtype=torch.int64, device=d)
        self.part_o = torch.empty(max_batch * self.H * self.splits * self.D, dtype=torch.float32, device=d)
        self.part_ml = torch.empty(max_batch * self.H * self.splits * 2, dtype=torch.float32, device=d)
        self.state = torch.zeros(max_batch, self.E, dtype=BF16, device=d)       # latent carried between tokens
        self.state_out = torch.zeros_like(self.state)
        self.init_buf = torch.zeros_like(self.state)                            # fresh random state per token
        self.tok_out = torch.zeros(max_batch, dtype=torch.int64, device=d)
        self.next_state = torch.zeros_like(self.state)
        self._seed = 1
        self.logits = torch.zeros(max_batch, self.V, dtype=torch.float32, device=d)
        self.prev_logp = torch.zeros_like(self.logits)
        self.kl = torch.zeros(max_batch, device=d)
        self.exited = torch.zeros(max_batch, dtype=torch.int32, device=d)
        self.prev_exited = torch.zeros_like(self.exited)
        self.steps_taken = torch.zeros(max_batch, dtype=torch.int32, device=d)
        self.live = torch.zeros(1, dtype=torch.int32, device=d)
        self._graphs: dict = {}
        self._qk_bias = {}
        self._norm_w: dict = {}
        # persistent fp32 accumulator of the stream-K skinny GEMMs (outputs up to the packed qkv width: qkv, attn.proj,
        # mlp.proj, adapter); kept zero between uses -- every consumer clears what it reads
        widest = max(2 * self.E, (self.H + 2 * self.Hkv) * self.D)
        if max_batch <= 16:  # narrow batches also accumulate the gate-up projection this way
            widest = max(widest, max(b.mlp.fc.weight.shape[0] for b in self._all_blocks()))
        self.work = torch.zeros(max_batch * widest, dtype=torch.float32, device=d)
        self.weight_bytes_per_recurrence = sum(p.numel() * 2 for n, p in model.named_parameters()
                                               if ".core_block." in n or ".adapter." in n)

    # -- kernels --------------------------------------------------------------------------------------
    def _linear(self, x, w, keep_f32: bool = False):
        """x [B, K] bf16 -> [B, N] through the skinny weight-streaming GEMM.  Narrow outputs are accumulated over K
        splits in the persistent fp32 ``work`` buffer (kept zero between uses by its consumers); ``keep_f32`` hands
        that buffer to a fused consumer, otherwise it is converted (and cleared) here."""
        Bt, Kd = x.shape
        N = w.shape[0]
        out = torch.empty(Bt, N, dtype=BF16, device=x.device)
        work = self.work[: Bt * N].view(Bt, N) if Bt * N <= self.work.numel() else None
        rc = _skinny(x.data_ptr(), w.data_ptr(), out.data_ptr(), K._ptr(work), Bt, N, Kd, x.stride(0), w.stride(0),
                     N, 0, K._stream(), K.err_word(x.device).data_ptr())
        K._launches += 1
        if rc < 0:
            raise RuntimeError(f"b200_gemm_skinny failed with code {rc}")
        if rc == 1:
            if keep_f32:
                return work
            K._check(_cast_zero(work.data_ptr(), out.data_ptr(), Bt * N, K._stream()), "cast_zero")
        return out

    def _all_blocks(self):
        t = self.model.transformer
        return list(t.prelude) + list(t.core_block) + list(t.coda)

    def _w(self, norm):
        """fp32 copy of a norm weight, made once."""
        key = id(norm)
        if key not in self._norm_w:
            self._norm_w[key] = None if norm.weight is None else norm.weight.detach().float().contiguous()
        return self._norm_w[key]

    def _pair(self, a, x, n1, n2=None):
        """y1 = n1(a + x), y2 = n2(y1) in one launch; ``a`` may be the fp32 split-K buffer, bf16, or None."""
        rows, E = (x if x is not None else a).shape
        y1 = torch.empty(rows, E, dtype=BF16, device=self.dev)
        y2 = torch.empty_like(y1) if n2 is not None else None
        K._check(_norm_pair(K._ptr(a), int(a is not None and a.dtype == torch.float32), K._ptr(x), K._ptr(self._w(n1)),
                            K._ptr(self._w(n2)) if n2 is not None else 0, y1.data_ptr(), K._ptr(y2), rows, E, n1.eps,
                            K._stream()), "add_rmsnorm_pair")
        return y1, y2

    def _bias(self, attn):
        key = id(attn)
        if key not in self._qk_bias:
            self._qk_bias[key] = None if attn.qk_bias is None else attn.qk_bias.detach().float().contiguous()
        return self._qk_bias[key]

    def _attention(self, attn, h, slot: int):
        B = h.shape[0]
        qkv = self._linear(h, attn.Wqkv.weight, keep_f32=True)   # bf16, or the fp32 stream-K accumulator
        q = torch.empty(B, self.H * self.D, dtype=BF16, device=h.device)
        kc, vc = self.cache.k[slot], self.cache.v[slot]
        bias = self._bias(attn)
        K._check(_rope_append(qkv.data_ptr(), K._ptr(bias), self.cos.data_ptr(), self.sin.data_ptr(),
                              self.pos.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, self.H, self.Hkv,
                              self.D, self.Lmax, K._stream(), int(qkv.dtype == torch.float32)), "rope_append")
        o = torch.empty_like(q)
        K._check(_decode_attn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), self.lens.data_ptr(), o.data_ptr(),
                              self.part_o.data_ptr(), self.part_ml.data_ptr(), B, self.H, self.Hkv, self.D, self.Lmax,
                              self.splits, float(self.D) ** -0.5, K._stream()), "decode_attention")
        return self._linear(o, attn.proj.weight, keep_f32=True)

    def _block(self, block, x, h, slot: int, next_norm=None):
        """Sandwich block on (residual x, h = norm_1(x)); returns (x', norm_1 of the next block applied to x')."""
        a = self._attention(block.attn, h, slot)
        x, h3 = self._pair(a, x, block.norm_2, block.norm_3)
        gu = self._linear(h3, block.mlp.fc.weight, keep_f32=True)
        if gu.dtype == torch.float32:
            g = torch.empty(gu.shape[0], gu.shape[1] // 2, dtype=BF16, device=self.dev)
            K._check(_swiglu_acc(gu.data_ptr(), g.data_ptr(), gu.shape[0], gu.shape[1] // 2, K._stream()), "swiglu_acc")
        else:
            g = K.swiglu_fwd(gu)
        m = self._linear(g, block.mlp.proj.weight, keep_f32=True)
        return self._pair(m, x, block.norm_4, next_norm)

    def _chain(self, blocks, x, slots, final_norm=None):
        """Run consecutive sandwich blocks, fusing each block's last norm with the next block's first."""
        h, _ = self._pair(None, x, blocks[0].norm_1)
        for i, block in enumerate(blocks):
            nxt = blocks[i + 1].norm_1 if i + 1 < len(blocks) else final_norm
            x, h = self._block(block, x, h, slots[i], nxt)
        return x, h

    def _embed(self):
        t = self.model.transformer
        e = K.embedding_fwd(self.tok, t.wte.weight, self.model.emb_scale)
        e, _ = self._chain(list(t.prelude), e, [self.cache.slot(i) for i in range(self.P)])
        return e

    def _recurrence(self, s, e, step: int):
        t = self.model.transformer
        s = self._linear(torch.cat([s, e], dim=-1), t.adapter.weight)
        slots = [self.cache.slot(self.P + self.R * step + b) for b in range(self.R)]
        s, _ = self._chain(list(t.core_block), s, slots)
        return s

    def _head(self, s):
        t = self.model.transformer
        x, _ = self._pair(None, s, t.ln_f)
        x, h = self._chain(list(t.coda), x, [self.cache.slot(-(i + 1)) for i in range(self.Cn)], final_norm=t.ln_f)
        lg = self._linear(h, self.model.lm_head.weight)
        B = lg.shape[0]
        self.logits[:B].copy_(lg)
        return self.logits[:B]

    # -- graph helpers ----------------------------------------------------------------------------------
    def _run(self, key, fn):
        """Replay ``fn`` as a CUDA graph.  ``fn`` must be idempotent (read inputs, write separate outputs): it is
        executed once eagerly as a warm-up and once more during capture before the first replay."""
        if not self.use_graphs:
            return self._with_pdl(fn)
        g = self._graphs.get(key)
        if g is None:
            self._with_pdl(fn)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = self._with_pdl(fn)
            g = self._graphs[key] = (graph, out)
        g[0].replay()
        return g[1]

    @staticmethod
    def _with_pdl(fn):
        """Run ``fn`` with programmatic dependent launch on for the decode kernels: each kernel's prologue overlaps the
        tail of its predecessor (the attribute is recorded into a graph at capture time)."""
        if not PDL:
            return fn()
        old = _set_pdl(1)
        try:
            return fn()
        finally:
            _set_pdl(old)

    def _fresh_state(self, init_scale: float):
        self._seed += 1
        std = self.cfg.init_values["std"] * init_scale * self.model.emb_scale
        if std <= 0:
            self.init_buf.zero_()
        else:
            self.init_buf.copy_(K.trunc_normal(self.init_buf.shape, std, self._seed, BF16, self.dev))

    # -- public API ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, num_steps: int | None = None, init_scale: float = 1.0):
        """Process the prompt with the ordinary (large-M) kernels, filling every cache slot; returns the first
        generated token and the last-position latent."""
        B, P = input_ids.shape
        assert B == self.B, "engine was built for a fixed batch"
        self.cache._seen_tokens = 0
        out = self.model(input_ids, num_steps=num_steps or self.r, use_cache=True, past_key_values=self.cache,
                         cache_position=torch.arange(P, device=self.dev), init_scale=init_scale)
        self.tok.copy_(out.logits[:, -1, :].argmax(-1))
        self.state.copy_(out.latent_states[:, -1, :])
        self.pos.fill_(P)
        self.lens.fill_(P + 1)
        return self.tok.clone()

    def _token_fixed(self, r: int, continuous: bool):
        """Graph body: token ``tok`` at position ``pos`` -> ``tok_out`` / ``state_out`` (inputs are not modified)."""
        e = self._embed()
        s = self.state if continuous else self.init_buf
        for step in range(r):
            s = self._recurrence(s, e, step)
        logits = self._head(s)
        self.state_out.copy_(s)
        self.tok_out.copy_(logits.argmax(-1))
        return self.tok_out

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, num_steps: int | None = None,
                 criterion: str | None = None, exit_threshold: float = 5e-4, max_steps: int | None = None,
                 continuous_compute: bool = False, init_scale: float = 1.0, check_every: int = 4, min_steps: int = 0):
        """Greedy decoding.  ``criterion=None``: fixed ``num_steps`` recurrences per token.  ``criterion="kl"``: KL
        exit with ``exit_threshold`` and at most ``max_steps`` recurrences.  Returns (tokens [B, P+new], stats)."""
        r = num_steps or self.r
        B, P = input_ids.shape
        assert P + max_new_tokens <= self.Lmax
        first = self.prefill(input_ids, r, init_scale)
        out = [first]
        steps_log = []
        if criterion is None:
            for _ in range(max_new_tokens - 1):
                if not continuous_compute:
                    self._fresh_state(init_scale)
                self._run(("fixed", r, continuous_compute), lambda: self._token_fixed(r, continuous_compute))
                self.tok.copy_(self.tok_out)
                self.state.copy_(self.state_out)
                self.pos.add_(1)
                self.lens.add_(1)
                out.append(self.tok.clone())
                steps_log.append([r] * B)
        else:
            assert criterion == "kl", "the device-side exit kernel implements the KL criterion"
            cap = max_steps or self.max_steps
            for _ in range(max_new_tokens - 1):
                out.append(self._token_adaptive(cap, exit_threshold, init_scale, continuous_compute, check_every,
                                                min_steps))
                steps_log.append(self.steps_taken.tolist())
        tokens = torch.cat([input_ids, torch.stack(out, dim=1)], dim=1)
        return tokens, {"steps": steps_log, "device_status": K.check_device_status()}

    def _token_adaptive(self, cap, threshold, init_scale, continuous, check_every, min_steps):
        B = self.B
        self.exited.zero_()
        self.prev_exited.zero_()
        self.steps_taken.zero_()
        self.live.fill_(B)
        self.prev_logp.fill_(-float(torch.log(torch.tensor(float(self.V)))))
        e = self._run(("embed",), self._embed)
        if not continuous:
            self._fresh_state(init_scale)
        self._s_buf = getattr(self, "_s_buf", torch.zeros_like(self.state))
        self._e_buf = getattr(self, "_e_buf", torch.zeros_like(self.state))
        self._s_buf.copy_(self.state if continuous else self.init_buf)
        self._e_buf.copy_(e)
        for step in range(cap):
            self._iter_step(step, threshold, armed=int(step >= min_steps))
            if (step + 1) % check_every == 0 or step == cap - 1:
                if int(self.live.item()) == 0:  # the only host read: every check_every recurrences
                    break
        self.state.copy_(self.next_state if continuous else self._s_buf)
        self.pos.add_(1)
        self.lens.add_(1)
        return self.tok.clone()

    def _iter_step(self, step: int, threshold: float, armed: int):
        def body():
            s = self._recurrence(self._s_buf, self._e_buf, step)
            self._s_buf.copy_(s)
            logits = self._head(s)
            K._check(_kl_exit(logits.data_ptr(), self.prev_logp.data_ptr(), self.kl.data_ptr(),
                              self.exited.data_ptr(), self.steps_taken.data_ptr(), self.tok.data_ptr(),
                              self.live.data_ptr(), self.B, self.V, float(threshold), step, armed, K._stream()),
                     "kl_exit")
            newly = (self.exited != self.prev_exited).unsqueeze(-1)
            self.next_state.copy_(torch.where(newly, s, self.next_state))
            self.prev_exited.copy_(self.exited)
            return s

        key = ("iter", step, float(threshold), armed)
        if self.use_graphs and key not in self._graphs:
            # capture without the warm-up side effects: snapshot and restore the mutable buffers
            snap = [t.clone() for t in (self._s_buf, self.prev_logp, self.exited, self.prev_exited, self.steps_taken,
                                        self.tok, self.live, self.next_state)]
            body()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = body()
            self._graphs[key] = (graph, out)
            for t, sv in zip((self._s_buf, self.prev_logp, self.exited, self.prev_exited, self.steps_taken, self.tok,
                              self.live, self.next_state), snap):
                t.copy_(sv)
        self._run(key, body)
