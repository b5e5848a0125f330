"""Training checkpoint -> HF-style folder (config.json + weights), with parity checks on the way.

Counterpart of evaluate_raven/checkpoint_to_hf_converter.py:85-193: load the raw training checkpoint, strip wrapper
prefixes from parameter names, build the inference model, compare its logits with the training implementation, check
that greedy generation with and without the KV cache agrees, then ``save_pretrained``.  There is no network here, so a
Hub upload is an explicit opt-in that simply calls ``push_to_hub`` and lets its error surface.

    python -m recurrent_pretraining_b200.evaluate.convert_to_hf CKPT.pth --out_dir outputs/hf/my_model
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch

from ..config import ModelConfig
from ..models.hf import RavenForCausalLM
from ..models.hf_config import RavenConfig
from ..runtime.checkpoint import strip_wrapper_prefixes


def load_training_checkpoint(path: str):
    """Returns (ModelConfig, state dict with clean names).  Accepts this framework's checkpoints and the reference's
    (``model_config`` stored as a dict with a registry ``name``; parameter names possibly carrying compile / wrapper
    prefixes)."""
    state = torch.load(path, map_location="cpu", weights_only=False, mmap=True)
    mc = state.get("model_config")
    if isinstance(mc, dict):
        name = mc.get("name")
        overrides = {k: v for k, v in mc.items() if k in ("block_size", "mean_recurrence", "mean_backprop_depth")}
        try:
            cfg = ModelConfig.from_name(name, **overrides)
        except Exception:
            cfg = ModelConfig.from_dict(mc)
    elif mc is not None:
        cfg = mc
    else:
        raise ValueError(f"{path} carries no model_config")
    sd = strip_wrapper_prefixes({k: v for k, v in state["model"].items() if "forward_module" not in k})
    return cfg, sd


@torch.no_grad()
def greedy(model, ids, max_new_tokens: int, num_steps: int, use_cache: bool):
    """Greedy continuation from a zero start state: through ``generate`` (KV cache) or by re-running the full sequence
    for every new token (no cache) -- the two must agree."""
    if use_cache:
        out = model.generate(ids, max_new_tokens=max_new_tokens, num_steps=num_steps, init_scale=0.0)
        return (out["sequences"] if isinstance(out, dict) else out)[0].tolist()
    for _ in range(max_new_tokens):
        logits = model(ids, num_steps=num_steps, init_scale=0.0).logits
        ids = torch.cat([ids, logits[:, -1:].argmax(-1)], dim=1)
    return ids[0].tolist()


def convert(checkpoint: str, out_dir: str, compare_to_pretrain_implementation: bool = True, num_steps: int | None = None,
            dtype: torch.dtype = torch.bfloat16, device: str = "cpu", upload_repo: str | None = None) -> dict:
    t0 = time.time()
    cfg, sd = load_training_checkpoint(checkpoint)
    hf = RavenForCausalLM(RavenConfig.from_model_config(cfg))
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    missing = [k for k in missing if "freqs_cis" not in k]
    if missing or unexpected:
        raise RuntimeError(f"state dict mismatch: missing {missing[:5]}, unexpected {unexpected[:5]}")
    hf = hf.to(device).eval()
    r = num_steps or cfg.mean_recurrence
    report = {"checkpoint": checkpoint, "params": sum(p.numel() for p in hf.parameters()), "num_steps": r}
    ids = torch.randint(0, cfg.vocab_size, (1, min(16, cfg.block_size // 2)), generator=torch.Generator().manual_seed(0))
    ids = ids.to(device)
    if compare_to_pretrain_implementation:
        train_model = cfg.construct_model().to(device).eval()
        train_model.load_state_dict(sd, strict=False)
        with torch.no_grad():
            states = torch.zeros(1, ids.shape[1], cfg.n_embd, device=device)
            a = train_model(ids, num_steps_pair=torch.tensor([r, 0]), input_states=states, return_logits=True)["logits"]
            b = hf(ids, num_steps=r, input_states=states).logits
        report["max_logit_diff_vs_training_model"] = float((a.float() - b.float()).abs().max())
    report["greedy_no_cache"] = greedy(hf, ids, 8, r, False)
    report["greedy_cache"] = greedy(hf, ids, 8, r, True)
    report["cache_consistent"] = report["greedy_no_cache"] == report["greedy_cache"]
    os.makedirs(out_dir, exist_ok=True)
    hf.to(dtype).save_pretrained(out_dir)
    with open(os.path.join(out_dir, "conversion_report.json"), "w") as f:
        json.dump(report, f, indent=1)
    if upload_repo:
        hf.push_to_hub(repo_id=upload_repo, private=True)
    report["seconds"] = round(time.time() - t0, 2)
    return report


def hf_implementation_test_and_upload(checkpoint_name: str, tokenizer_path: str | None = None, device="cpu",
                                      out_dir: str = "outputs/eval", upload: bool = False,
                                      compare_to_pretrain_implementation: bool = False,
                                      hf_gen_crosscheck: bool = False) -> dict:
    """The reference's entry point (evaluate_raven/checkpoint_to_hf_converter.py:85-193): convert
    ``checkpoint_name`` into ``<out_dir>/<checkpoint stem>``, copy the tokenizer files beside the weights when a local
    tokenizer folder is given, optionally compare against the training implementation; ``hf_gen_crosscheck`` is always
    done (cached against uncached greedy decoding).  ``upload`` pushes to a Hub repository named like the checkpoint
    and needs network access."""
    import os
    import shutil

    model_name = str(checkpoint_name).split("/")[-1].split(".")[0]
    target = os.path.join(out_dir, model_name)
    report = convert(checkpoint_name, target, compare_to_pretrain_implementation, dtype=torch.bfloat16
                     if str(device).startswith("cuda") else torch.float32, device=str(device),
                     upload_repo=model_name if upload else None)
    if tokenizer_path and os.path.isdir(tokenizer_path):
        for name in os.listdir(tokenizer_path):
            if name.startswith(("tokenizer", "special_tokens", "added_tokens", "vocab", "merges")):
                shutil.copy(os.path.join(tokenizer_path, name), target)
    return report


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("checkpoint")
    ap.add_argument("--out_dir", default="outputs/hf_model")
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--num_steps", type=int, default=None)
    ap.add_argument("--no_compare", action="store_true")
    ap.add_argument("--upload_repo", default=None)
    a = ap.parse_args(argv)
    print(json.dumps(convert(a.checkpoint, a.out_dir, not a.no_compare, a.num_steps, device=a.device,
                             upload_repo=a.upload_repo), indent=1))


if __name__ == "__main__":
    main()
