"""Worker for tests/test_cpu_distributed.py (gloo, one process per rank)."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline"))

from recurrent_pretraining_b200.config import ModelConfig  # noqa: E402
from recurrent_pretraining_b200.parallel.fabric import Fabric  # noqa: E402
from recurrent_pretraining_b200.runtime.engine import TrainEngine  # noqa: E402

OV = dict(state_init="zero")
STEPS = 6


def batches(rank, vocab):
    g = torch.Generator().manual_seed(0 + 1000 * rank)
    return [torch.randint(0, vocab, (2, 257), generator=g) for _ in range(STEPS)]


def parity():
    import refload

    fabric = Fabric.from_env(backend="gloo", grad_sync="chunked")
    torch.manual_seed(0)
    cfg = ModelConfig.from_name("tiny-raven-cpu", **OV)
    model = cfg.construct_model()
    ref_model, _ = refload.build_train_model("tiny-raven-cpu" if False else "nebel-raven-3.5b", **{
        **dict(block_size=256, vocab_size=8192, padding_multiple=512, n_embd=256, num_attention_heads=4,
               num_key_value_heads=4, intermediate_size=704, n_layers_in_recurrent_block=2, n_layers_in_prelude=1,
               n_layers_in_coda=1, mean_recurrence=4, mean_backprop_depth=2), **OV})
    ref_model.load_state_dict(model.state_dict())
    eng = TrainEngine(model, fabric, lr=4e-4, mode="torch")
    ours = []
    data = batches(fabric.global_rank, cfg.padded_vocab_size)
    for ids in data:
        ours.append(eng.train_step(ids[:, :-1], ids[:, 1:])["loss"].item())
    # the reference's own pieces: its model, param groups, AdamW, chunked all-reduce, clipping, first-step skip
    ro, ru = refload.module("optim"), refload.module("utils")
    groups = ro.get_param_groups(ref_model.named_parameters(), no_weight_decay_for_bias_and_norm_params=False)
    opt = torch.optim.AdamW(groups, lr=4e-4, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8)
    theirs, ref_model = [], ref_model.train()
    for step, ids in enumerate(data):
        ref_model.step = step + 1
        loss = ref_model(ids[:, :-1].contiguous(), labels=ids[:, 1:].contiguous())["loss"]
        loss.backward()
        ru._allreduce_chunk_stream(ref_model, fabric.world_size, torch.device("cpu"))
        gn = torch.nn.utils.clip_grad_norm_(ref_model.parameters(), 1.0)
        if torch.isfinite(gn) and step > 0:
            opt.step()
        opt.zero_grad()
        theirs.append(loss.item())
    theirs_p = dict(ref_model.named_parameters())
    diff = max((p - theirs_p[n]).abs().max().item() for n, p in model.named_parameters())
    # replicas stay identical across ranks
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    other = flat.clone()
    dist.broadcast(other, 0)
    if fabric.global_rank == 0:
        print("RESULT " + json.dumps({"ours": ours, "theirs": theirs, "param_diff": diff}))
    same = torch.tensor([float(torch.equal(flat, other))])
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    if fabric.global_rank == 0:
        print("RESULT2 " + json.dumps({"replicas_identical": bool(same.item())}))
    fabric.shutdown()


def rank_failure():
    """Rank 1 dies on the host before the collective; rank 0 must get an error from a bounded wait, not hang."""
    import datetime

    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo", rank=rank, world_size=int(os.environ["WORLD_SIZE"]),
                            timeout=datetime.timedelta(seconds=8))
    t = torch.ones(4)
    dist.all_reduce(t)
    if rank == 1:
        os._exit(17)  # leaves between steps with nothing in flight
    try:
        dist.all_reduce(t)
        print("RESULT " + json.dumps({"error": None}))
    except Exception as exc:  # noqa: BLE001
        print("RESULT " + json.dumps({"error": type(exc).__name__}))
    os._exit(0)


def exit_flag():
    """The cooperative exit flag is MIN-reduced: training stops only once every rank raised it."""
    fabric = Fabric.from_env(backend="gloo")
    out = []
    for raised in ([1.0, 0.0], [1.0, 1.0]):
        flag = torch.tensor([raised[fabric.global_rank]])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        out.append(bool(flag.item()))
    if fabric.global_rank == 0:
        print("RESULT " + json.dumps({"stop": out}))
    fabric.shutdown()


def tensor_parallel():
    """Two-way tensor parallel model against the unsharded model: same loss, gradient shards equal slices."""
    import copy

    from recurrent_pretraining_b200.parallel.tensor_parallel import gather_full_weight, tensor_parallelize

    fabric = Fabric.from_env(backend="gloo", grad_sync="chunked")
    rank, tp = fabric.global_rank, fabric.world_size
    torch.manual_seed(0)
    cfg = ModelConfig.from_name("tiny-raven-cpu", **OV)
    full = cfg.construct_model()
    sharded = tensor_parallelize(copy.deepcopy(full))
    ids = torch.randint(0, cfg.padded_vocab_size, (2, 65), generator=torch.Generator().manual_seed(5))
    pair = torch.tensor([1, 2])
    a = full(ids[:, :-1], labels=ids[:, 1:], num_steps_pair=pair)["loss"]
    b = sharded(ids[:, :-1], labels=ids[:, 1:], num_steps_pair=pair)["loss"]
    a.backward()
    b.backward()
    fp, sp = dict(full.named_parameters()), dict(sharded.named_parameters())
    name = "transformer.core_block.0.attn.Wqkv.weight"
    H, D, E = cfg.n_head, cfg.n_embd // cfg.n_head, cfg.n_embd
    h = H // tp
    want = torch.cat([fp[name].grad[sec * H * D:(sec + 1) * H * D].view(H, D, E)[rank * h:(rank + 1) * h].reshape(h * D, E)
                      for sec in range(3)], 0)
    g_qkv = (sp[name].grad - want).abs().max().item()
    name2 = "transformer.core_block.1.mlp.proj.weight"
    I = cfg.intermediate_size // tp
    g_proj = (sp[name2].grad - fp[name2].grad[:, rank * I:(rank + 1) * I]).abs().max().item()
    g_norm = (sp["transformer.ln_f.weight"].grad - fp["transformer.ln_f.weight"].grad).abs().max().item()
    g_emb = (sp["transformer.wte.weight"].grad - fp["transformer.wte.weight"].grad).abs().max().item()
    gathered = gather_full_weight(sp[name2].data, dim=1)
    out = {"loss_full": a.item(), "loss_tp": b.item(), "g_qkv": g_qkv, "g_proj": g_proj, "g_norm": g_norm, "g_emb": g_emb,
           "gather_ok": bool(torch.equal(gathered, fp[name2].data)),
           "params_local": sum(p.numel() for p in sharded.parameters()), "params_full": sum(p.numel() for p in full.parameters())}
    if rank == 0:
        print("RESULT " + json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


def _train(fabric, flags, steps=5, accum=1):
    torch.manual_seed(0)
    cfg = ModelConfig.from_name("tiny-raven-cpu", **OV)
    model = cfg.construct_model()
    eng = TrainEngine(model, fabric, lr=2e-3, weight_decay=0.05, eps=1e-6, mode="fused", grad_accum=accum, **flags)
    losses, norms = [], []
    g = torch.Generator().manual_seed(7 + 1000 * fabric.global_rank)
    for i in range(steps * accum):
        ids = torch.randint(0, cfg.padded_vocab_size, (2, 65), generator=g)
        out = eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([1, 2]))
        losses.append(out["loss"].item())
        if out["grad_norm"] is not None:
            norms.append(float(out["grad_norm"]))
    params = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    return eng, losses, norms, params


def sharded_step():
    """The sharded optimizer step (per-tensor ownership, buckets fired from the model's phase hooks, sharded moments)
    on gloo collectives against the replicated flat path, for AdamW and for the ELLISAdam flags; then the parameter-
    sharded layout and the re-cut of a two-rank optimizer checkpoint for one rank."""
    from recurrent_pretraining_b200.optim.fused import FusedAdamW
    from recurrent_pretraining_b200.parallel.flat import flatten_group
    from recurrent_pretraining_b200.parallel.p2p import ShardedStepper

    fabric = Fabric.from_env(backend="gloo", grad_sync="p2p-host")
    plain = Fabric(fabric.device, fabric.global_rank, fabric.world_size, fabric.local_rank, "chunked")
    out = {}
    ellis = dict(atan2=True, update_clipping=True, running_init=True, decouple_wd=True)
    for tag, flags, accum in (("adamw", {}, 1), ("ellis", ellis, 1), ("accum", {}, 2)):
        e1, l1, n1, p1 = _train(fabric, flags, accum=accum)
        fired = {b.name for b in e1.fabric._p2p.buckets.values()}
        e2, l2, n2, p2 = _train(plain, flags, accum=accum)
        out[tag] = {"loss_diff": max(abs(a - b) for a, b in zip(l1, l2)),
                    "norm_diff": max(abs(a - b) for a, b in zip(n1, n2)),
                    "param_diff": (p1 - p2).abs().max().item(), "buckets": sorted(fired),
                    "state_numel": sum(g.state["m"].numel() for g in e1.flat_groups),
                    "full_numel": sum(g.state["m"].numel() for g in e2.flat_groups)}
        if tag == "ellis":
            sharded_sd, full_opt = e1.state_dict(), e2.optimizer
    # re-cut: both ranks' optimizer state -> a replicated (unsharded) optimizer
    both = [None, None]
    dist.all_gather_object(both, sharded_sd)
    want = [(g.state["m"].clone(), g.state["v"].clone()) for g in full_opt.groups]
    fresh = FusedAdamW(full_opt.groups, **ellis)        # replaces the groups' moments by zeros of full size
    fresh.load_state_dict(both[fabric.global_rank]["optimizer"], lambda: [b["optimizer"] for b in both])
    out["recut_diff"] = max(max((g.state["m"] - m).abs().max().item(), (g.state["v"] - v).abs().max().item())
                            for g, (m, v) in zip(fresh.groups, want))

    # parameter-sharded layout: synthetic gradients, one update, against the replicated result
    torch.manual_seed(3)
    shapes = {"transformer.coda.0.attn.Wqkv.weight": (48, 16), "transformer.core_block.0.mlp.fc.weight": (64, 16),
              "transformer.prelude.0.attn.proj.weight": (16, 16), "transformer.adapter.weight": (16, 32)}
    vals = {k: torch.randn(*v) for k, v in shapes.items()}
    grads = {k: torch.randn(*v) for k, v in shapes.items()}

    def build(shard):
        params = [torch.nn.Parameter(v.clone()) for v in vals.values()]
        g = flatten_group(params, list(shapes), torch.device("cpu"), True, {"lr": 1e-2, "base_lr": 1.0,
                                                                           "weight_decay": 0.1}, shard=shard)
        for p, k in zip(params, shapes):
            p.grad.copy_(grads[k])
        return g

    gs = build((fabric.world_size, fabric.global_rank))
    opt_s = FusedAdamW([gs], lr=1e-2)
    st = ShardedStepper(fabric, [gs], opt_s, None, zero3=True, backend="torch")
    for b in st.buckets.values():
        b.fired = True
    st.master_sharded = [True]
    st._step_torch(opt_s, 1.0, 1.0 / fabric.world_size, True)
    gr = build(None)
    gr.grad.mul_(fabric.world_size)
    opt_r = FusedAdamW([gr], lr=1e-2)
    opt_r.step(max_norm=1.0, grad_scale=1.0 / fabric.world_size)
    out["zero3_shadow_diff"] = (gs.shadow.float() - gr.shadow.float()).abs().max().item()
    full = st.full_master(0, 1)
    out["zero3_master_diff"] = (full - gr.master[gr.offsets[1]:gr.offsets[1] + full.numel()].view_as(full)).abs().max().item()
    out["zero3_master_numel"] = [gs.master.numel(), gr.master.numel()]
    if fabric.global_rank == 0:
        print("RESULT " + json.dumps(out))
    fabric.shutdown()


def ddp_alternative():
    """torch DistributedDataParallel as the gradient sync against the hand-rolled chunked all-reduce: same losses and
    parameters, with accumulation (no_sync) and the untracked recurrences (unused-parameter detection)."""
    out = {}
    runs = {}
    for sync in ("chunked", "ddp"):
        fabric = Fabric.from_env(backend="gloo", grad_sync=sync)
        torch.manual_seed(0)
        cfg = ModelConfig.from_name("tiny-raven-cpu", **OV)
        model = cfg.construct_model()
        eng = TrainEngine(model, fabric, lr=1e-3, mode="torch", grad_accum=2)
        g = torch.Generator().manual_seed(11 + 1000 * fabric.global_rank)
        losses = []
        for i in range(6):
            ids = torch.randint(0, cfg.padded_vocab_size, (2, 65), generator=g)
            losses.append(eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor([1, 2]))["loss"].item())
        runs[sync] = (losses, torch.cat([p.detach().reshape(-1) for p in model.parameters()]), eng)
    out["loss_diff"] = max(abs(a - b) for a, b in zip(runs["chunked"][0], runs["ddp"][0]))
    out["param_diff"] = (runs["chunked"][1] - runs["ddp"][1]).abs().max().item()
    out["wrapped"] = type(runs["ddp"][2].ddp).__name__
    if dist.get_rank() == 0:
        print("RESULT " + json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    {"parity": parity, "rank_failure": rank_failure, "exit_flag": exit_flag,
     "tensor_parallel": tensor_parallel, "sharded_step": sharded_step, "ddp_alternative": ddp_alternative}[sys.argv[1]]()
