"""Serving layer on top of the decode engine: request batching + an OpenAI-style HTTP API, one replica per GPU.

Role of the reference's vLLM plugin (vllm/raven_vllm.py:297-411 fixed-recurrence model, :471-542 weight loading,
vllm/README.md:19-24 data-parallel replicas).  That plugin is a library path (vLLM's scheduler, attention and paged
cache) with a fixed recurrence; here the product is the native engine (`engine/decode.py`): per-step static KV cache,
CUDA-graphed recurrence, latent reuse and device-side KL exit, so the adaptive-depth options are served too.

Pieces:
  * ``EngineBackend``  — a ``DecodeEngine`` on one GPU (bf16).
  * ``ModelBackend``   — the plain model ``generate`` path (any device; what the CPU tests use).
  * ``BatchScheduler`` — thread-safe queue; a worker groups waiting requests that share prompt length and decoding
                         options into one batch (up to ``max_batch``, waiting at most ``window_ms`` for company).
  * ``create_app``     — FastAPI app: ``/health``, ``/v1/models``, ``/v1/completions``.
"""
from __future__ import annotations

import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass
class DecodeOptions:
    max_tokens: int = 64
    num_steps: Optional[int] = None
    criterion: Optional[str] = None          # None = fixed depth, "kl" = adaptive exit
    exit_threshold: float = 5e-4
    max_steps: Optional[int] = None
    continuous_compute: bool = False
    init_scale: float = 1.0                  # multiplies the sigma of the random start state (0 = deterministic)

    def key(self):
        return (self.max_tokens, self.num_steps, self.criterion, self.exit_threshold, self.max_steps,
                self.continuous_compute, self.init_scale)


@dataclass
class Request:
    prompt_ids: list
    options: DecodeOptions
    id: str = field(default_factory=lambda: "cmpl-" + uuid.uuid4().hex[:24])
    done: threading.Event = field(default_factory=threading.Event)
    tokens: Optional[list] = None
    steps: Optional[list] = None
    error: Optional[str] = None
    t_enqueue: float = field(default_factory=time.time)
    t_done: float = 0.0


class ModelBackend:
    """Decoding through the model's own ``generate`` (greedy).  Works on CPU; batch rows are independent."""

    def __init__(self, model, max_batch: int = 8):
        self.model, self.max_batch = model.eval(), max_batch
        self.device = next(model.parameters()).device
        self.name = "model.generate"

    @torch.no_grad()
    def generate(self, prompts: list, opt: DecodeOptions):
        ids = torch.tensor(prompts, dtype=torch.long, device=self.device)
        kwargs = dict(max_new_tokens=opt.max_tokens, num_steps=opt.num_steps, continuous_compute=opt.continuous_compute,
                      init_scale=opt.init_scale)
        if opt.criterion:
            kwargs.update(criterion=opt.criterion, exit_threshold=opt.exit_threshold)
        kwargs = {k: v for k, v in kwargs.items() if v is not None}
        out = self.model.generate(ids, **kwargs)
        seq = out["sequences"] if isinstance(out, dict) else out
        return [row[len(p):].tolist() for row, p in zip(seq, prompts)], None


class EngineBackend:
    """The native decode engine on one GPU.  The engine's buffers are sized for ``max_batch`` rows; smaller batches are
    padded by repeating the first prompt and the padding rows are dropped from the result."""

    def __init__(self, model, max_batch: int = 8, max_len: int = 4096, max_steps: int | None = None,
                 cache_lookup_strategy: str = "full"):
        from .decode import DecodeEngine

        self.engine = DecodeEngine(model, max_batch=max_batch, max_len=max_len, max_steps=max_steps,
                                   cache_lookup_strategy=cache_lookup_strategy)
        self.max_batch, self.device = max_batch, self.engine.dev
        self.name = "decode-engine"

    @torch.no_grad()
    def generate(self, prompts: list, opt: DecodeOptions):
        rows = prompts + [prompts[0]] * (self.max_batch - len(prompts))
        ids = torch.tensor(rows, dtype=torch.long, device=self.device)
        tokens, stats = self.engine.generate(ids, opt.max_tokens, num_steps=opt.num_steps, criterion=opt.criterion,
                                             exit_threshold=opt.exit_threshold, max_steps=opt.max_steps,
                                             continuous_compute=opt.continuous_compute, init_scale=opt.init_scale)
        if stats.get("device_status"):
            raise RuntimeError(f"decode kernels reported device status {stats['device_status']}")
        P = len(prompts[0])
        steps = None
        if stats.get("steps"):
            steps = [[per_tok[i] for per_tok in stats["steps"]] for i in range(len(prompts))]
        return [tokens[i, P:].tolist() for i in range(len(prompts))], steps


class BatchScheduler:
    def __init__(self, backend, window_ms: float = 3.0, stop_ids=(65504, 65505, 65508)):
        self.backend, self.window = backend, window_ms / 1e3
        self.stop_ids = set(stop_ids)
        self.q: "queue.Queue[Request]" = queue.Queue()
        self.stats = {"requests": 0, "batches": 0, "tokens": 0, "busy_s": 0.0}
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, name="decode-batcher", daemon=True)
        self._thread.start()

    def submit(self, prompt_ids: list, options: DecodeOptions) -> Request:
        req = Request(list(prompt_ids), options)
        self.q.put(req)
        return req

    def close(self):
        self._stop.set()
        self._thread.join(timeout=5)

    def _collect(self):
        """One batch: the oldest request plus whatever compatible ones arrive within the window."""
        try:
            first = self.q.get(timeout=0.1)
        except queue.Empty:
            return None
        batch, rest = [first], []
        deadline = time.time() + self.window
        while len(batch) < self.backend.max_batch:
            try:
                r = self.q.get(timeout=max(0.0, deadline - time.time()))
            except queue.Empty:
                break
            same = len(r.prompt_ids) == len(first.prompt_ids) and r.options.key() == first.options.key()
            (batch if same else rest).append(r)
        for r in rest:  # incompatible requests go back, in order, for the next round
            self.q.put(r)
        return batch

    def _truncate(self, toks: list) -> list:
        for i, t in enumerate(toks):
            if t in self.stop_ids:
                return toks[:i + 1]
        return toks

    def _loop(self):
        while not self._stop.is_set():
            batch = self._collect()
            if not batch:
                continue
            t0 = time.time()
            try:
                outs, steps = self.backend.generate([r.prompt_ids for r in batch], batch[0].options)
                for i, r in enumerate(batch):
                    r.tokens = self._truncate(outs[i])
                    r.steps = steps[i][:len(r.tokens)] if steps else None
            except Exception as e:  # the request carries the failure; the server keeps running
                for r in batch:
                    r.error = f"{type(e).__name__}: {e}"
            dt = time.time() - t0
            self.stats["requests"] += len(batch)
            self.stats["batches"] += 1
            self.stats["busy_s"] += dt
            self.stats["tokens"] += sum(len(r.tokens or []) for r in batch)
            for r in batch:
                r.t_done = time.time()
                r.done.set()


def completion_payload(req: Request, model_name: str, text: Optional[str]) -> dict:
    return {"id": req.id, "object": "text_completion", "created": int(req.t_enqueue), "model": model_name,
            "choices": [{"index": 0, "text": text, "token_ids": req.tokens, "finish_reason": "stop"
                         if req.tokens and len(req.tokens) < req.options.max_tokens else "length",
                         "recurrence_steps": req.steps}],
            "usage": {"prompt_tokens": len(req.prompt_ids), "completion_tokens": len(req.tokens or []),
                      "total_tokens": len(req.prompt_ids) + len(req.tokens or [])},
            "latency_s": round(req.t_done - req.t_enqueue, 4)}


def handle_completion(scheduler: BatchScheduler, body: dict, tokenizer=None, model_name: str = "raven",
                      timeout_s: float = 600.0) -> dict:
    """Framework-independent request handler (the FastAPI route and the tests both call this)."""
    prompt = body.get("prompt")
    if isinstance(prompt, str):
        if tokenizer is None:
            raise ValueError("a text prompt needs a tokenizer; send token ids instead")
        ids = tokenizer.encode(prompt)
        ids = ids.tolist() if hasattr(ids, "tolist") else list(ids)
    elif isinstance(prompt, list) and prompt and all(isinstance(t, int) for t in prompt):
        ids = prompt
    else:
        raise ValueError("prompt must be a string or a non-empty list of token ids")
    opt = DecodeOptions(max_tokens=int(body.get("max_tokens", 64)), num_steps=body.get("num_steps"),
                        criterion=body.get("criterion"), exit_threshold=float(body.get("exit_threshold", 5e-4)),
                        max_steps=body.get("max_steps"), continuous_compute=bool(body.get("continuous_compute", False)),
                        init_scale=float(body.get("init_scale", 1.0)))
    req = scheduler.submit(ids, opt)
    if not req.done.wait(timeout_s):
        raise TimeoutError("generation timed out")
    if req.error:
        raise RuntimeError(req.error)
    text = tokenizer.decode(req.tokens) if tokenizer is not None and hasattr(tokenizer, "decode") else None
    return completion_payload(req, model_name, text)


def create_app(scheduler: BatchScheduler, tokenizer=None, model_name: str = "raven"):
    from fastapi import FastAPI, HTTPException
    from fastapi.concurrency import run_in_threadpool

    app = FastAPI(title="recurrent-depth LM server")

    @app.get("/health")
    def health():
        return {"status": "ok", "backend": scheduler.backend.name, **scheduler.stats}

    @app.get("/v1/models")
    def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model"}]}

    @app.post("/v1/completions")
    async def completions(body: dict):
        try:
            return await run_in_threadpool(handle_completion, scheduler, body, tokenizer, model_name)
        except ValueError as e:
            raise HTTPException(status_code=400, detail=str(e))
        except (RuntimeError, TimeoutError) as e:
            raise HTTPException(status_code=500, detail=str(e))

    return app
