#!/usr/bin/env python
"""Serve a recurrent-depth model over HTTP with the native decode engine, one replica per GPU.

    python serve.py --model /path/to/hf_folder --port 8000                # one GPU
    python serve.py --model nebel-raven-3.5b --random-init --replicas 8   # 8 replicas on ports 8000..8007 + router on 7999

``--replicas N`` starts N child processes (replica i pinned to GPU i via CUDA_VISIBLE_DEVICES) and a round-robin router
in the parent: inference data parallelism, the deployment shape of the reference's vLLM recipe (vllm/README.md:19-24).
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import subprocess
import sys
import urllib.request


def load_model(name: str, random_init: bool, device, dtype):
    import torch

    from recurrent_pretraining_b200.models.hf import RavenForCausalLM
    from recurrent_pretraining_b200.models.hf_config import RavenConfig

    if os.path.isdir(name):
        return RavenForCausalLM.from_pretrained(name, torch_dtype=dtype).to(device)
    if not random_init:
        raise SystemExit(f"{name!r} is not a local folder; pass --random-init to serve a registry shape with random weights")
    from recurrent_pretraining_b200.config import ModelConfig

    torch.manual_seed(0)
    with torch.device(device):
        model = RavenForCausalLM(RavenConfig.from_model_config(ModelConfig.from_name(name)))
    return model.to(dtype)


def run_replica(args):
    import torch
    import uvicorn

    from recurrent_pretraining_b200.engine.server import BatchScheduler, EngineBackend, ModelBackend, create_app

    cuda = torch.cuda.is_available() and not args.cpu
    device = torch.device("cuda", 0) if cuda else torch.device("cpu")
    model = load_model(args.model, args.random_init, device, torch.bfloat16 if cuda else torch.float32)
    tokenizer = None
    if args.tokenizer:
        from recurrent_pretraining_b200.data.tokenizer import Tokenizer

        tokenizer = Tokenizer(args.tokenizer)
    backend = (EngineBackend(model, args.max_batch, args.max_len, args.max_steps, args.cache_lookup_strategy)
               if cuda else ModelBackend(model, args.max_batch))
    sched = BatchScheduler(backend, window_ms=args.batch_window_ms)
    uvicorn.run(create_app(sched, tokenizer, os.path.basename(args.model.rstrip("/"))), host=args.host, port=args.port,
                log_level="warning")


def run_router(args, ports):
    """Round-robin forwarder for /v1/completions; /health aggregates the replicas."""
    import uvicorn
    from fastapi import FastAPI, HTTPException
    from fastapi.concurrency import run_in_threadpool

    cycle = itertools.cycle(ports)
    app = FastAPI(title="replica router")

    def forward(port, path, body=None):
        req = urllib.request.Request(f"http://127.0.0.1:{port}{path}", method="POST" if body is not None else "GET",
                                     data=None if body is None else json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=900) as r:
            return json.loads(r.read())

    @app.get("/health")
    async def health():
        out = {}
        for p in ports:
            try:
                out[str(p)] = await run_in_threadpool(forward, p, "/health")
            except Exception as e:
                out[str(p)] = {"status": f"unreachable: {e}"}
        return out

    @app.post("/v1/completions")
    async def completions(body: dict):
        try:
            return await run_in_threadpool(forward, next(cycle), "/v1/completions", body)
        except Exception as e:
            raise HTTPException(status_code=502, detail=str(e))

    uvicorn.run(app, host=args.host, port=args.port - 1, log_level="warning")


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="local HF folder or a registry shape name (with --random-init)")
    ap.add_argument("--random-init", action="store_true")
    ap.add_argument("--tokenizer", default=None, help="local tokenizer folder (text prompts); token-id prompts need none")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--replicas", type=int, default=1)
    ap.add_argument("--max-batch", type=int, default=8)
    ap.add_argument("--max-len", type=int, default=4096)
    ap.add_argument("--max-steps", type=int, default=None, help="recurrence cap the KV cache is sized for")
    ap.add_argument("--cache-lookup-strategy", default="full")
    ap.add_argument("--batch-window-ms", type=float, default=3.0)
    ap.add_argument("--cpu", action="store_true", help="serve through model.generate on CPU (debug)")
    ap.add_argument("--replica-index", type=int, default=None, help=argparse.SUPPRESS)
    args = ap.parse_args(argv)
    if args.replicas <= 1 or args.replica_index is not None:
        return run_replica(args)
    ports, children = [], []
    base = [a for a in (argv or sys.argv[1:])]
    try:
        for i in range(args.replicas):
            port = args.port + i
            ports.append(port)
            env = dict(os.environ, CUDA_VISIBLE_DEVICES=str(i))
            cmd = [sys.executable, os.path.abspath(__file__)] + base + ["--replica-index", str(i), "--port", str(port)]
            children.append(subprocess.Popen(cmd, env=env))
        print(f"replicas on ports {ports}; router on {args.port - 1}", flush=True)
        run_router(args, ports)
    finally:
        for c in children:
            c.terminate()
        for c in children:
            c.wait(timeout=30)


if __name__ == "__main__":
    main()
