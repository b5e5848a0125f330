"""Per-kernel time shares of one flagship training step (torch.profiler / CUPTI; shares only, never a bench value).

``python -m recurrent_pretraining_b200.utils.step_profile [model] [n] [k]`` prints the kernels of one step with
fixed recurrence (n, k), grouped by name and sorted by device time.
"""
from __future__ import annotations

import sys

import torch
from torch.profiler import ProfilerActivity, profile

from ..config import ModelConfig
from ..runtime.engine import TrainEngine


def main():
    name = sys.argv[1] if len(sys.argv) > 1 else "nebel-raven-3.5b"
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 24
    k = int(sys.argv[3]) if len(sys.argv) > 3 else 8
    cfg = ModelConfig.from_name(name)
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    with torch.device(dev):
        model = cfg.construct_model()
    eng = TrainEngine(model, lr=4e-4, skip_first_step=False)
    S = cfg.block_size
    ids = torch.randint(0, cfg.padded_vocab_size, (1, S + 1), device=dev)
    pair = torch.tensor([n, k])
    for _ in range(2):
        out = eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=pair)
    torch.cuda.synchronize()
    print("loss", float(out["loss"]), "grad_norm", float(out["grad_norm"]))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=pair)
    e1.record()
    torch.cuda.synchronize()
    print(f"unprofiled step: {e0.elapsed_time(e1):.1f} ms; model TFLOP {cfg.flops_per_token(S, n, k) * S / 1e12:.1f}")
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=pair)
        torch.cuda.synchronize()
    rows = [e for e in prof.key_averages() if e.device_time_total > 0 and e.device_type.name == "CUDA"]
    rows.sort(key=lambda e: -e.device_time_total)
    total = sum(e.device_time_total for e in rows)
    print(f"total kernel time {total / 1e3:.1f} ms")
    for e in rows[:40]:
        print(f"{e.device_time_total / 1e3:9.2f} ms {100 * e.device_time_total / total:5.1f}%  x{e.count:5d}  {e.key[:110]}")
    # idle time between consecutive kernels: where the device waited for the host
    kern = sorted((e for e in prof.events() if e.device_type.name == "CUDA" and e.device_time_total > 0),
                  key=lambda e: e.time_range.start)
    if kern:
        span = (kern[-1].time_range.end - kern[0].time_range.start) / 1e3
        gaps = []
        end = kern[0].time_range.end
        prev = kern[0]
        for e in kern[1:]:
            if e.time_range.start > end:
                gaps.append(((e.time_range.start - end) / 1e3, prev.name[:60], e.name[:60]))
            if e.time_range.end > end:
                end, prev = e.time_range.end, e
        idle = sum(g[0] for g in gaps)
        print(f"first-to-last kernel span {span:.1f} ms, idle inside it {idle:.2f} ms in {len(gaps)} gaps")
        for g in sorted(gaps, reverse=True)[:8]:
            print(f"  gap {g[0]:7.3f} ms after {g[1]} before {g[2]}")


if __name__ == "__main__":
    main()
