#!/usr/bin/env python
"""Self-speculative decoding with one recurrent model (script form of the reference's spec_decoding_example.ipynb):
draft a few tokens with a shallow recurrence, verify all of them in one deep forward, keep the agreeing prefix.

    python examples/speculative_decoding_demo.py
"""
from __future__ import annotations

import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from examples.inference_demo import tiny_model  # noqa: E402


def main():
    model = tiny_model()
    ids = torch.randint(0, model.config.vocab_size, (1, 12), generator=torch.Generator().manual_seed(1))
    r = model.config.mean_recurrence
    t0 = time.time()
    plain = model.generate(ids, max_new_tokens=24, num_steps=r, init_scale=0.0)
    t_plain = time.time() - t0
    print(f"plain      num_steps={r}: {t_plain:5.2f}s  {plain[0, 12:].tolist()}")
    for draft, look in ((max(1, r // 4), 4), (max(1, r // 2), 8)):
        t0 = time.time()
        spec = model.generate(ids, max_new_tokens=24, num_steps=r, draft_steps=draft, lookahead_for_draft=look,
                              init_scale=0.0)
        dt = time.time() - t0
        same = spec[0, :36].tolist() == plain[0, :36].tolist()
        print(f"draft {draft:2d} x{look}: {dt:5.2f}s ({t_plain / dt:4.2f}x)  identical to plain greedy: {same}")


if __name__ == "__main__":
    main()
