"""Probe: can a small classifier tell from a latent state how many recurrences produced it?

Counterpart of scripts/classify_loops.py: run the HF-style model on token batches, capture the latent state after every
recurrence, and train a gated-MLP classifier (over all depths, or one-vs-next binary problems) on them.  A probe that
stays at chance means consecutive iterations are indistinguishable, i.e. the recurrence has converged."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


@torch.no_grad()
def capture_latents(model, input_ids: torch.Tensor, num_steps: int, init_scale: float = 1.0) -> torch.Tensor:
    """[num_steps, B, S, E] latent states of the recurrent core after 1 .. num_steps iterations."""
    embeds, block_idx = model.embed_inputs(input_ids)
    state = model.initialize_state(embeds, scale=init_scale)
    out, step = [], torch.tensor(0)
    for i in range(num_steps):
        state, block_idx, step = model.iterate_one_step(embeds, state, block_idx=block_idx, current_step=step)
        out.append(state.float().clone())
    return torch.stack(out)


class LoopClassifier(nn.Module):
    def __init__(self, n_embd: int, n_classes: int, hidden: int = 0):
        super().__init__()
        hidden = hidden or 2 * n_embd
        self.norm = nn.LayerNorm(n_embd)
        self.fc = nn.Linear(n_embd, 2 * hidden)
        self.proj = nn.Linear(hidden, n_embd)
        self.head = nn.Linear(n_embd, n_classes)

    def forward(self, x):
        h = self.norm(x)
        a, b = self.fc(h).chunk(2, dim=-1)
        return self.head(h + self.proj(F.silu(a) * b))


def probe_loss(clf: LoopClassifier, latents: torch.Tensor, classes: torch.Tensor | None = None):
    """Cross entropy of predicting the depth index of every token latent; ``classes`` selects / relabels depths
    (e.g. ``tensor([3, 4])`` for a binary problem between depths 3 and 4)."""
    steps = torch.arange(latents.shape[0]) if classes is None else classes
    x = latents[steps].flatten(1, 2)                     # [C, B*S, E]
    y = torch.arange(len(steps)).repeat_interleave(x.shape[1])
    logits = clf(x.flatten(0, 1))
    return F.cross_entropy(logits, y.to(logits.device)), (logits.argmax(-1).cpu() == y).float().mean().item()


def train_probe(model, batches, num_steps: int, classes=None, lr: float = 1e-3, hidden: int = 0) -> dict:
    """Train on every batch of ``batches`` (token id tensors); returns the accuracy trace and the chance level."""
    n_classes = num_steps if classes is None else len(classes)
    clf = LoopClassifier(model.config.n_embd, n_classes, hidden)
    opt = torch.optim.AdamW(clf.parameters(), lr=lr)
    accs = []
    for ids in batches:
        lat = capture_latents(model, ids, num_steps)
        loss, acc = probe_loss(clf, lat, classes)
        opt.zero_grad()
        loss.backward()
        opt.step()
        accs.append(acc)
    return {"accuracy": accs, "chance": 1.0 / n_classes, "classifier": clf}


def binary_sweep(model, make_batches, num_steps: int, gap: int = 1, **kw) -> dict:
    """One binary probe per pair (d, d + gap): where along the recurrence do states stop being separable?"""
    return {d: train_probe(model, make_batches(), num_steps, classes=torch.tensor([d, d + gap]), **kw)["accuracy"][-1]
            for d in range(0, num_steps - gap)}
