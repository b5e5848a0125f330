"""Worker run under torch.distributed.run by tests/test_gpu_multi.py (one process per GPU)."""
import copy
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from recurrent_pretraining_b200.config import ModelConfig  # noqa: E402
from recurrent_pretraining_b200.parallel.fabric import Fabric  # noqa: E402
from recurrent_pretraining_b200.runtime.engine import TrainEngine  # noqa: E402


ELLIS = dict(atan2=True, update_clipping=True, running_init=True, decouple_wd=True)
DEPTHS = [(1, 2), (0, 3), (2, 1), (1, 2), (3, 1), (0, 2)]    # (n, k) varies from step to step, as with the sampler


def run_training(fabric, steps: int = 6, flags=None, accum: int = 1):
    torch.manual_seed(0)
    cfg = ModelConfig.from_name("smoke-raven-96", lockstep_n=True, lockstep_k=True)
    with torch.device(fabric.device):
        model = cfg.construct_model()
    eng = TrainEngine(model, fabric, lr=1e-3, eps=1e-6, grad_accum=accum, **(flags or {}))
    g = torch.Generator().manual_seed(100 + fabric.global_rank)
    losses, norms = [], []
    for i in range(steps * accum):
        ids = torch.randint(0, cfg.padded_vocab_size, (2, 129), generator=g).to(fabric.device)
        state = (torch.randn(2, 128, cfg.n_embd, generator=g) * 0.6).to(fabric.device).bfloat16()
        out = eng.train_step(ids[:, :-1], ids[:, 1:], num_steps_pair=torch.tensor(DEPTHS[(i // accum) % len(DEPTHS)]),
                             input_states=state)
        losses.append(out["loss"].item())
        if out["grad_norm"] is not None:
            norms.append(out["grad_norm"].item())
    fabric.sync_parameters()
    torch.cuda.synchronize()
    shadow = torch.cat([g_.shadow.float().cpu() for g_ in eng.flat_groups])
    return eng, losses, norms, shadow


def compare_modes(sync: str, flags=None, accum: int = 1):
    """The sharded step (``sync``) against the NCCL all-reduce + replicated update on the same data."""
    from recurrent_pretraining_b200.ops import cuda as K

    fabric = Fabric.from_env(grad_sync=sync)
    eng, l1, n1, s1 = run_training(fabric, flags=flags, accum=accum)
    status = K.check_device_status()
    mine = s1.to(fabric.device)
    ref = mine.clone()
    dist.broadcast(ref, 0)
    same = torch.tensor([float(torch.equal(mine, ref))], device=fabric.device)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    st = fabric._p2p
    info = {"overlap_fired": sorted(b.name for b in st.buckets.values()), "bytes": st.persistent_bytes(),
            "ag_weights": sum(1 for g_ in eng.flat_groups for p in g_.params if hasattr(p, "_ag"))}
    # checkpoint view of the fp32 parameters (collective): must equal the replicated run's masters
    sd = eng.model_state_dict()
    st.close()
    fabric._p2p = None
    fabric2 = Fabric(fabric.device, fabric.global_rank, fabric.world_size, fabric.local_rank, "flat")
    eng2, l2, n2, s2 = run_training(fabric2, flags=flags, accum=accum)
    sd2 = eng2.model_state_dict()
    master_rel = max(((sd[k].float() - sd2[k].float()).norm() / (sd2[k].float().norm() + 1e-12)).item()
                     for k in sd2 if k != "freqs_cis")
    rel = ((s1 - s2).norm() / s2.norm()).item()
    return fabric, {"losses": l1, "nccl_losses": l2, "norms": n1, "nccl_norms": n2,
                    "replicas_identical": bool(same.item()), "param_rel_diff": rel, "master_rel_diff": master_rel,
                    "status": status, **info}


def main():
    mode = sys.argv[1]
    from recurrent_pretraining_b200.ops import cuda as K

    if mode in ("train", "train_ellis", "train_accum", "zero3", "zero3_ellis"):
        sync = "zero3" if mode.startswith("zero3") else "p2p"
        flags = ELLIS if mode.endswith("ellis") else None
        fabric, res = compare_modes(sync, flags, accum=2 if mode == "train_accum" else 1)
        if fabric.global_rank == 0:
            print("RESULT " + json.dumps(res))
        dist.barrier()
        dist.destroy_process_group()
    elif mode == "tensor_parallel":
        # two-way tensor parallel blocks on the CUDA kernels (NCCL all-reduces) against the unsharded model
        from recurrent_pretraining_b200.parallel.tensor_parallel import tensor_parallelize

        fabric = Fabric.from_env(grad_sync="flat")
        dev, rank, tp = fabric.device, fabric.global_rank, fabric.world_size
        torch.manual_seed(0)
        cfg = ModelConfig.from_name("smoke-raven-96", n_embd=384, num_attention_heads=4, num_key_value_heads=4, intermediate_size=1024)
        full = cfg.construct_model()
        sharded = tensor_parallelize(copy.deepcopy(full))
        full, sharded = full.to(dev).bfloat16(), sharded.to(dev).bfloat16()
        ids = torch.randint(0, cfg.padded_vocab_size, (2, 129), generator=torch.Generator().manual_seed(5)).to(dev)
        state = (torch.randn(2, 128, cfg.n_embd, generator=torch.Generator().manual_seed(6)) * 0.6).to(dev).bfloat16()
        pair = torch.tensor([1, 2])
        a = full(ids[:, :-1], labels=ids[:, 1:], num_steps_pair=pair, input_states=state)["loss"]
        b = sharded(ids[:, :-1], labels=ids[:, 1:], num_steps_pair=pair, input_states=state)["loss"]
        a.backward()
        b.backward()
        torch.cuda.synchronize()
        fp, sp = dict(full.named_parameters()), dict(sharded.named_parameters())

        def rel(x, y):
            return ((x.float() - y.float()).norm() / (y.float().norm() + 1e-12)).item()

        name = "transformer.core_block.0.attn.Wqkv.weight"
        H, D, E = cfg.n_head, cfg.n_embd // cfg.n_head, cfg.n_embd
        h = H // tp
        want = torch.cat([fp[name].grad[sec * H * D:(sec + 1) * H * D].view(H, D, E)[rank * h:(rank + 1) * h]
                          .reshape(h * D, E) for sec in range(3)], 0)
        name2 = "transformer.core_block.1.mlp.proj.weight"
        i = cfg.intermediate_size // tp
        res = {"loss_full": a.item(), "loss_tp": b.item(), "g_qkv": rel(sp[name].grad, want),
               "g_proj": rel(sp[name2].grad, fp[name2].grad[:, rank * i:(rank + 1) * i]),
               "g_norm": rel(sp["transformer.ln_f.weight"].grad, fp["transformer.ln_f.weight"].grad),
               "g_emb": rel(sp["transformer.wte.weight"].grad, fp["transformer.wte.weight"].grad),
               "status": K.check_device_status()}
        worst = torch.tensor([res["g_qkv"], res["g_proj"], res["g_norm"], res["g_emb"]], device=dev)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        res["g_qkv"], res["g_proj"], res["g_norm"], res["g_emb"] = worst.tolist()
        if rank == 0:
            print("RESULT " + json.dumps(res))
        dist.barrier()
        dist.destroy_process_group()
    elif mode == "collectives":
        # one-launch fused collectives on bf16 buckets against torch sums
        from recurrent_pretraining_b200.parallel.collectives import FusedCollectives
        from recurrent_pretraining_b200.parallel.symm import SymmetricBuffer

        fabric = Fabric.from_env(grad_sync="flat")
        dev, rank, N = fabric.device, fabric.global_rank, fabric.world_size
        out = {}
        fc = FusedCollectives(fabric, 1 << 20)
        shadow = SymmetricBuffer(fabric, fc.max_elems * 2)
        for count in (8 * N, 40000, 1 << 20):
            gen = torch.Generator().manual_seed(50 + count)
            all_data = [(torch.randn(count, generator=gen) * 1e-3).bfloat16() for _ in range(N)]
            want = sum(d.float() for d in all_data) / N
            fc.bucket[:count].copy_(all_data[rank])
            case = {}
            for one_shot in (True, False):
                res = fc.all_reduce(count, 1.0 / N, one_shot=one_shot).float().cpu()
                torch.cuda.synchronize()
                case[f"allreduce_oneshot{int(one_shot)}"] = (res - want).abs().max().item()
                norm_sq = fc.partial.clone()
                if not one_shot:
                    dist.all_reduce(norm_sq)
                case[f"norm_oneshot{int(one_shot)}"] = abs(norm_sq.sqrt().item() - want.norm().item()) / want.norm().item()
            lo, hi = fc.my_slice(count)
            rs = fc.reduce_scatter(count, 1.0 / N).float().cpu()
            torch.cuda.synchronize()
            case["reduce_scatter"] = (rs - want[lo:hi]).abs().max().item() if hi > lo else 0.0
            # all-gather: every rank contributes its slice of its own bucket
            mine = torch.full((count,), float(rank + 1)).bfloat16()
            fc.bucket[:count].copy_(mine)
            torch.cuda.synchronize()
            dist.barrier()
            got = fc.all_gather_bf16(count).float().cpu()
            torch.cuda.synchronize()
            per = fc.slice_elems(count)
            exp = torch.cat([torch.full((min(per, max(count - q * per, 0)),), float(q + 1)) for q in range(N)])
            case["all_gather"] = (got - exp).abs().max().item()
            # reduce-scatter + AdamW + push against torch
            fc.bucket[:count].copy_(all_data[rank])
            p0 = torch.randn(count, generator=torch.Generator().manual_seed(7))
            p = p0[lo:hi].clone().to(dev)
            m, v = torch.zeros_like(p), torch.zeros_like(p)
            torch.cuda.synchronize()
            dist.barrier()
            gn = fc.reduce_scatter_adamw(count, p, m, v, shadow, lr=1e-2, eps=1e-8, weight_decay=0.1, step=1,
                                         max_norm=1e-3, scale=1.0 / N)
            torch.cuda.synchronize()
            dist.barrier()
            gnorm = want.norm().item()
            clip = min(1.0, 1e-3 / (gnorm + 1e-6))
            g = want * clip
            mm = 0.1 * g
            vv = 0.05 * g * g
            pref = p0 * (1 - 1e-2 * 0.1) - 1e-2 / 0.1 * mm / (vv.sqrt() / (0.05 ** 0.5) + 1e-8)
            sh = shadow.tensor(torch.bfloat16, count).float().cpu()
            case["adamw_gnorm"] = abs(gn.item() - gnorm) / gnorm
            case["adamw_shadow"] = (sh - pref).abs().max().item()
            case["adamw_master"] = (p.cpu() - pref[lo:hi]).abs().max().item() if hi > lo else 0.0
            out[str(count)] = case
        status = K.check_device_status()
        if rank == 0:
            print("RESULT " + json.dumps({"cases": out, "status": status}))
        dist.barrier()
        shadow.close()
        fc.close()
        dist.destroy_process_group()
    elif mode == "timeout":
        # a barrier whose peer flag nobody sets must give up and report through the status word
        import ctypes as C

        from recurrent_pretraining_b200.parallel.symm import SymmetricBuffer

        fabric = Fabric.from_env(grad_sync="flat")
        ctrl = SymmetricBuffer(fabric, 512)
        torch.cuda.synchronize()
        dist.barrier()
        code = 0
        if fabric.global_rank == 0:  # only rank 0 enters: its peer never signals epoch 7
            K._check(K.lib.b200_barrier(ctrl.ptr_array(0), 0, fabric.world_size, C.c_uint(7), 200, None, None,
                                        C.c_void_p(K.err_word(fabric.device).data_ptr()), C.c_void_p(K._stream())),
                     "barrier")
            torch.cuda.synchronize()
            code = K.check_device_status()
            x = torch.ones(4, device=fabric.device) * 2  # the context is still usable
            print("RESULT " + json.dumps({"status": code, "after": float(x.sum())}))
        dist.barrier()
        ctrl.close()
        dist.destroy_process_group()
    elif mode == "ag_gemm":
        # all-gather fused into the GEMM: result and gathered weight against the plain library path
        from recurrent_pretraining_b200.parallel.ag_gemm import GatheredWeight

        fabric = Fabric.from_env(grad_sync="flat")
        dev = fabric.device
        out = {}
        for (M, N, Kd) in ((512, 1440, 264), (1024, 2000, 528)):
            torch.manual_seed(1)
            w = (torch.randn(N, Kd, device=dev) * 0.2).bfloat16()      # identical on every rank (same seed)
            x = torch.randn(M, Kd, device=dev).bfloat16()
            gw = GatheredWeight(fabric, N, Kd)
            gw.load_full(w)
            torch.cuda.synchronize()
            dist.barrier()                                              # every shard is in place
            y = gw.gemm(x)
            torch.cuda.synchronize()
            dist.barrier()
            want = x.float() @ w.float().T
            err = ((y.float() - want).abs().max() / want.abs().max()).item()
            out[f"{M}x{N}x{Kd}"] = {"rel_err": err, "weight_equal": bool(torch.equal(gw.full, w)),
                                    "second_call_equal": bool(torch.equal(gw.gemm(x), y))}
            gw.close()
        status = K.check_device_status()
        if fabric.global_rank == 0:
            print("RESULT " + json.dumps({"cases": out, "status": status}))
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
