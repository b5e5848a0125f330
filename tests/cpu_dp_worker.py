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


if __name__ == "__main__":
    {"parity": parity, "rank_failure": rank_failure, "exit_flag": exit_flag,
     "tensor_parallel": tensor_parallel}[sys.argv[1]]()
