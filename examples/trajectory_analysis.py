#!/usr/bin/env python
"""Latent-state trajectories over the recurrence (script form of the reference's trajectory_analysis.ipynb).

For every token of a prompt the core block is iterated step by step from a random start state; the script records the
latent after every step and reports, per token: how fast the state converges (norm of the step-to-step change), whether
it settles into a fixed point, a slow drift or an orbit (cosine between successive changes), and the coordinates of the
trajectory in the plane of its first two principal components (written to a CSV that any plotting tool can read).

    python examples/trajectory_analysis.py --steps 32 --out trajectories.csv
"""
from __future__ import annotations

import argparse
import csv
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from examples.inference_demo import tiny_model  # noqa: E402
from recurrent_pretraining_b200.models.hf import RavenForCausalLM  # noqa: E402


@torch.no_grad()
def latent_trajectories(model, ids: torch.Tensor, steps: int, init_scale: float = 1.0) -> torch.Tensor:
    """[steps + 1, T, E]: the state of every position after 0..steps recurrences (whole sequence at once)."""
    e, block_idx = model.embed_inputs(ids)
    x = model.initialize_state(e, scale=init_scale)
    out = [x[0].float().cpu()]
    for s in range(steps):
        x, block_idx, _ = model.iterate_one_step(e, x, block_idx=block_idx, current_step=s)
        out.append(x[0].float().cpu())
    return torch.stack(out)


def analyse(traj: torch.Tensor) -> list[dict]:
    """Per-token convergence statistics and 2-D PCA coordinates of the trajectory."""
    steps, T, E = traj.shape
    rows = []
    for t in range(T):
        z = traj[:, t]                                   # [steps, E]
        d = z[1:] - z[:-1]
        dn = d.norm(dim=-1)
        cos = torch.nn.functional.cosine_similarity(d[1:], d[:-1], dim=-1) if len(d) > 1 else torch.zeros(1)
        tail = dn[-max(2, len(dn) // 4):]
        ratio = float(tail.mean() / dn[0].clamp_min(1e-12))
        kind = "fixed point" if ratio < 0.05 else ("orbit" if float(cos[-len(tail):].mean()) < 0.0 else "slow drift")
        zc = z - z.mean(0, keepdim=True)
        _, _, v = torch.pca_lowrank(zc, q=2, center=False)
        xy = zc @ v[:, :2]
        rows.append({"token": t, "first_change": float(dn[0]), "last_change": float(dn[-1]), "tail_ratio": ratio,
                     "tail_cosine": float(cos[-len(tail):].mean()), "behaviour": kind, "xy": xy.tolist()})
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default=None, help="local HF folder; a tiny random model otherwise")
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--out", default=None, help="CSV with the PCA coordinates per token and step")
    a = ap.parse_args(argv)
    model = RavenForCausalLM.from_pretrained(a.model).eval() if a.model else tiny_model()
    ids = torch.randint(0, model.config.vocab_size, (1, a.tokens), generator=torch.Generator().manual_seed(3))
    traj = latent_trajectories(model, ids, a.steps)
    rows = analyse(traj)
    for r in rows:
        print(f"token {r['token']:2d}: |dz| {r['first_change']:8.3f} -> {r['last_change']:8.3f}  "
              f"(ratio {r['tail_ratio']:.3f}, cosine {r['tail_cosine']:+.2f})  {r['behaviour']}")
    if a.out:
        with open(a.out, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["token", "step", "pc1", "pc2"])
            for r in rows:
                for s, (x, y) in enumerate(r["xy"]):
                    w.writerow([r["token"], s, x, y])
        print(f"wrote {a.out}")
    return rows


if __name__ == "__main__":
    main()
