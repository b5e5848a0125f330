"""Fused optimizer kernels on one GPU against the Python optimizers they restate."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _groups(device, shapes):
    from recurrent_pretraining_b200.parallel.flat import flatten_group

    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(*s) * 0.1) for s in shapes]
    names = [f"transformer.core_block.0.w{i}.weight" for i in range(len(shapes))]
    ref = [torch.nn.Parameter(p.detach().clone()) for p in params]
    g = flatten_group(params, names, device, True, {"lr": 3e-3, "base_lr": 1.0, "weight_decay": 0.05})
    return g, params, ref


@pytest.mark.parametrize("flags", [
    dict(atan2=True, update_clipping=True, running_init=True, decouple_wd=True),     # the production combination
    dict(atan2=False, update_clipping=True, running_init=False, decouple_wd=True),
    dict(atan2=True, update_clipping=False, running_init=True, decouple_wd=False),
])
def test_fused_ellis_flags_match_the_python_optimizer(flags):
    """Five steps of the table-driven update kernel (per-tensor clipping statistics, running init, atan2, decoupled
    decay) against ``optim.ellis.ELLISAdam``, which the CPU tests pin to the reference's ELLISAdam."""
    from recurrent_pretraining_b200.optim.ellis import ELLISAdam
    from recurrent_pretraining_b200.optim.fused import FusedAdamW

    dev = torch.device("cuda")
    shapes = [(96, 64), (264, 40), (8,), (4096, 33 * 4)]
    g, params, ref = _groups(dev, shapes)
    fused = FusedAdamW([g], lr=3e-3, betas=(0.9, 0.95), eps=1e-6, weight_decay=0.05, **flags)
    py = ELLISAdam(ref, lr=3e-3, betas=(0.9, 0.95), eps=1e-6, weight_decay=0.05, atan_adam=flags["atan2"],
                   update_clipping=flags["update_clipping"], running_init=flags["running_init"],
                   decouple_wd=flags["decouple_wd"])
    gen = torch.Generator().manual_seed(1)
    for step in range(5):
        lr = 3e-3 * (0.5 + 0.1 * step)
        for h in fused.param_groups:
            h["lr"] = lr
        for grp in py.param_groups:
            grp["lr"] = torch.tensor(lr)
        for p, r in zip(params, ref):
            grad = torch.randn(p.shape, generator=gen) * (10.0 if step == 2 else 0.3)   # one step trips the clipping
            p.grad.copy_(grad)
            r.grad = grad.clone()
        fused.step(max_norm=0.0, grad_scale=1.0, zero_grad=False)
        py.step()
    torch.cuda.synchronize()
    for p, r, off in zip(params, ref, g.offsets):
        got = g.master[off:off + p.numel()].view(p.shape).cpu()
        assert torch.allclose(got, r.detach(), rtol=2e-4, atol=2e-6), (p.shape, (got - r.detach()).abs().max())
        lp = g.shadow[off:off + p.numel()].view(p.shape).float().cpu()
        assert torch.allclose(lp, r.detach(), rtol=1e-2, atol=1e-3)


def test_table_update_equals_plain_adamw_kernel():
    """The table-driven kernel with no ELLIS flag set is AdamW: same result as the flat AdamW kernel."""
    from recurrent_pretraining_b200.optim.fused import FusedAdamW
    from recurrent_pretraining_b200.parallel.p2p import single_device_table_step

    dev = torch.device("cuda")
    shapes = [(128, 96), (40,), (1000, 8)]
    ga, pa, _ = _groups(dev, shapes)
    gb, pb, _ = _groups(dev, shapes)
    oa = FusedAdamW([ga], lr=1e-3, eps=1e-8, weight_decay=0.1)
    ob = FusedAdamW([gb], lr=1e-3, eps=1e-8, weight_decay=0.1)
    gen = torch.Generator().manual_seed(2)
    for step in range(3):
        for p, q in zip(pa, pb):
            grad = torch.randn(p.shape, generator=gen)
            p.grad.copy_(grad)
            q.grad.copy_(grad)
        oa.step(max_norm=1.0, grad_scale=0.5, zero_grad=False)
        ob.compute_grad_norm_sq()
        first = ob.step_count == 0
        ob.step_count += 1
        single_device_table_step(ob, 1.0, 0.5, False, first)
    torch.cuda.synchronize()
    assert torch.allclose(ga.master, gb.master, rtol=1e-6, atol=1e-8)
    assert torch.equal(ga.shadow, gb.shadow)
    # the table kernel keeps its state packed per tensor (no alignment gaps); compare tensor by tensor
    from recurrent_pretraining_b200.parallel.segments import GroupShards

    plan = GroupShards.plan(gb, 1)
    for off, so, n in zip(plan.offs, plan.state_offsets(0), plan.numels):
        for key in ("m", "v"):
            a, b = ga.state[key][off:off + n], gb.state[key][so:so + n]
            # m sums signed terms (cancellation: absolute bound at its 1e-3 scale); v is a sum of squares
            assert torch.allclose(a, b, rtol=1e-4, atol=1e-8 if key == "m" else 1e-12), (key, (a - b).abs().max().item())


@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (1000, 136, 264), (5280, 5280, 1024)])
def test_fp32_products_on_split_bf16_tensor_cores(M, N, K):
    """fp32 x fp32 on three bf16 tcgen05 GEMMs (hi*hi + hi*lo + lo*hi): all four operand layouts against float64."""
    from recurrent_pretraining_b200.ops import cuda as C

    gen = torch.Generator().manual_seed(M + N)
    a = torch.randn(M, K, generator=gen).cuda()
    b = torch.randn(N, K, generator=gen).cuda()
    want = (a.double() @ b.double().T)
    scale = want.abs().max().item()
    for a_mn in (False, True):
        for b_mn in (False, True):
            aa = a.T.contiguous() if a_mn else a
            bb = b.T.contiguous() if b_mn else b
            got = C.matmul_f32(aa, bb, a_mn=a_mn, b_mn=b_mn)
            err = (got.double() - want).abs().max().item() / scale
            assert err < 3e-5, (a_mn, b_mn, err)
    # one bf16 GEMM alone is two orders of magnitude worse: the split is what buys the accuracy
    one = C.gemm(a.bfloat16(), b.bfloat16(), out_mode=C.OUT_F32)
    assert (one.double() - want).abs().max().item() / scale > 3e-4
    assert C.check_device_status() == 0


def test_soap_step_on_tensor_cores_matches_cpu():
    """SOAP on CUDA parameters (its Gram matrices and rotations on the split-bf16 GEMMs) against the same optimizer on
    the CPU (torch.tensordot): same parameters after a few steps."""
    from recurrent_pretraining_b200.optim.soap import SOAP

    gen = torch.Generator().manual_seed(0)
    # square: both Gram matrices of a random gradient have full rank, so the eigenbases are determined up to signs
    # (which the update does not depend on)
    w0 = torch.randn(256, 256, generator=gen) * 0.1
    grads = [torch.randn(256, 256, generator=gen) * 0.05 for _ in range(4)]
    outs = []
    for dev in ("cpu", "cuda"):
        p = torch.nn.Parameter(w0.clone().to(dev))
        opt = SOAP([p], lr=1e-2, precondition_frequency=2, weight_decay=0.0)
        for g in grads:
            p.grad = g.to(dev)
            opt.step()
        outs.append(p.detach().cpu())
    assert (outs[0] - outs[1]).abs().max().item() < 5e-3 * outs[0].abs().max().item()
