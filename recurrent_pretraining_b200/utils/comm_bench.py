"""Communication sweep: fused NVLink kernels vs NCCL on gradient buckets of 1 MB .. 1 GB.

Run under ``python -m torch.distributed.run --nproc-per-node N -m recurrent_pretraining_b200.utils.comm_bench``.
Device-timed with CUDA events, max over ranks, median of 10.

Default sweep (bf16 buckets drawn N(0, 1e-3^2)): for every size the one-launch fused collectives of
``parallel/collectives.py`` -- all-reduce (bf16 in, fp32 cast + 1/N scale + squared-norm partial, result on every rank),
reduce-scatter, all-gather, and reduce-scatter + clipped AdamW + bf16 parameter push -- each beside the NCCL call that
the reference's path would make (``all_reduce`` on bf16 and on fp32, ``reduce_scatter_tensor``,
``all_gather_into_tensor``).  A row's roofline time is the bytes that must cross one GPU's NVLink in one direction
(its own traffic plus what it serves to its peers) divided by the link bandwidth; fractions are given against the measured 770 GB/s per direction and against
the nominal 900 GB/s.  ``--fp32`` adds the older fp32 two-shot sequence, ``--phases`` the per-phase CTA sweep, ``--ag``
the all-gather fused into the GEMM.
"""
from __future__ import annotations

import ctypes as C
import json
import statistics
import sys

import torch
import torch.distributed as dist

from ..parallel.fabric import Fabric
from ..parallel.symm import SymmetricBuffer

LINK_GBS = 770.0       # measured peer copy, per direction
LINK_NOMINAL = 900.0   # NVLink 5, per direction


def _time(fn, device, reps=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    ts = []
    for _ in range(reps):
        dist.barrier(device_ids=[device.index])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(device)
        t = torch.tensor([e0.elapsed_time(e1)], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts.append(float(t))
    return statistics.median(ts)


def bf16_sweep(fabric, sizes_mb) -> None:
    """bf16 buckets: fused one-launch collectives against NCCL (see the module docstring)."""
    from ..ops import cuda as K
    from ..parallel.collectives import FusedCollectives

    dev, rank, N = fabric.device, fabric.global_rank, fabric.world_size
    max_elems = max(sizes_mb) * 2**20 // 2
    fc = FusedCollectives(fabric, max_elems)
    shadow = SymmetricBuffer(fabric, fc.max_elems * 2)
    fc.bucket.normal_(0, 1e-3)
    nccl_bf16 = torch.empty(max_elems, dtype=torch.bfloat16, device=dev).normal_(0, 1e-3)
    nccl_f32 = torch.empty(max_elems, dtype=torch.float32, device=dev).normal_(0, 1e-3)
    per_max = fc.slice_elems(max_elems)
    p = torch.zeros(per_max, device=dev)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    torch.cuda.synchronize(dev)
    dist.barrier(device_ids=[dev.index])
    f = (N - 1) / N
    for mb in sizes_mb:
        count = mb * 2**20 // 2
        nb = count * 2
        lo, hi = fc.my_slice(count)
        per = fc.slice_elems(count)
        rows = []
        # (name, ours, nccl, bytes over this GPU's link per direction).  Every direction carries both what this GPU
        # asks for and what its peers ask of it: the all-reduce sends its fp32 slice results out (f * count * 4) while
        # serving the peers' reads of its bf16 bucket (f * count * 2), and receives the mirror image.
        ar_bytes = f * count * 6
        rows.append(("all_reduce bf16->fp32 (+scale, norm)", lambda: fc.all_reduce(count, 1.0 / N, one_shot=False),
                     lambda: dist.all_reduce(nccl_f32[:count]), ar_bytes, "nccl all_reduce fp32"))
        if nb <= 64 * 2**20:
            rows.append(("all_reduce one-shot", lambda: fc.all_reduce(count, 1.0 / N, one_shot=True),
                         lambda: dist.all_reduce(nccl_bf16[:count]), (N - 1) * nb, "nccl all_reduce bf16"))
        rows.append(("reduce_scatter bf16->fp32 (+scale, norm)", lambda: fc.reduce_scatter(count, 1.0 / N),
                     lambda: dist.reduce_scatter_tensor(nccl_bf16[:per], nccl_bf16[:per * N]) if per * N <= max_elems
                     else dist.all_reduce(nccl_bf16[:count]), f * nb, "nccl reduce_scatter bf16"))
        rows.append(("all_gather bf16 (push)", lambda: fc.all_gather_bf16(count),
                     lambda: dist.all_gather_into_tensor(nccl_bf16[:per * N], nccl_bf16[:per]) if per * N <= max_elems
                     else dist.all_reduce(nccl_bf16[:count]), f * nb, "nccl all_gather bf16"))

        def nccl_update():
            dist.reduce_scatter_tensor(nccl_f32[:per], nccl_f32[:per * N]) if per * N <= max_elems else None
            g = nccl_f32[:hi - lo]
            torch.nn.utils.clip_grad_norm_([g], 1.0) if False else g.norm()
            m[:hi - lo].lerp_(g, 0.1)
            v[:hi - lo].mul_(0.95).addcmul_(g, g, value=0.05)
            p[:hi - lo].mul_(1 - 4e-5).addcdiv_(m[:hi - lo], v[:hi - lo].sqrt().add_(1e-8), value=-4e-4)
            nccl_bf16[:hi - lo].copy_(p[:hi - lo])
            dist.all_gather_into_tensor(nccl_bf16[:per * N], nccl_bf16[:per]) if per * N <= max_elems else None

        rows.append(("reduce_scatter + clip + AdamW + bf16 push",
                     lambda: fc.reduce_scatter_adamw(count, p[:hi - lo], m[:hi - lo], v[:hi - lo], shadow, lr=4e-4,
                                                     step=2, scale=1.0 / N),
                     nccl_update, 2 * f * nb, "nccl reduce_scatter fp32 + torch AdamW + all_gather bf16"))
        for name, ours, theirs, link_bytes, nccl_name in rows:
            t_ours = _time(ours, dev)
            t_nccl = _time(theirs, dev)
            gbs = link_bytes / t_ours / 1e6
            rec = {"bucket_MB": mb, "dtype": "bf16", "n_gpus": N, "op": name, "ms": round(t_ours, 4),
                   "link_GBps": round(gbs, 1), "frac_of_measured_link": round(gbs / LINK_GBS, 3),
                   "frac_of_nominal_link": round(gbs / LINK_NOMINAL, 3), "nccl": nccl_name,
                   "nccl_ms": round(t_nccl, 4), "speedup_vs_nccl": round(t_nccl / t_ours, 2)}
            if rank == 0:
                print(json.dumps(rec), flush=True)
    status = K.check_device_status()
    if rank == 0:
        print(json.dumps({"bf16_sweep_device_status": status}), flush=True)
    torch.cuda.synchronize(dev)
    dist.barrier(device_ids=[dev.index])
    shadow.close()
    fc.close()


def main():
    from ..ops import cuda as K

    fabric = Fabric.from_env(grad_sync="flat")
    dev, rank, N = fabric.device, fabric.global_rank, fabric.world_size
    sizes_mb = [1, 4, 16, 64, 256, 1024]
    if "--sizes" in sys.argv:
        sizes_mb = [int(x) for x in sys.argv[sys.argv.index("--sizes") + 1].split(",")]
    max_bytes = max(sizes_mb) * 2**20
    if "--ag-only" not in sys.argv and "--fp32-only" not in sys.argv:
        bf16_sweep(fabric, sizes_mb)
    if "--fp32" not in sys.argv and "--fp32-only" not in sys.argv:
        sizes_mb = []
    if "--ag-only" in sys.argv:   # only the fused all-gather GEMM rows
        sizes_mb = []
    buf = SymmetricBuffer(fabric, max_bytes + 4096 * N)  # slack: slices are rounded up to 512 B
    ctrl = SymmetricBuffer(fabric, 512)
    out = torch.empty(max_bytes // 4, dtype=torch.float32, device=dev)
    sumsq = torch.zeros(1, device=dev)
    src_f32 = buf.tensor(torch.float32, max_bytes // 4)
    src_f32.normal_(0, 1e-3)
    epoch = [0]
    flags = ctrl.ptr_array(0)
    err = C.c_void_p(K.err_word(dev).data_ptr())

    def barrier():
        epoch[0] += 1
        K._check(K.lib.b200_barrier(flags, rank, N, C.c_uint(epoch[0]), 20000, None, None, err,
                                    C.c_void_p(K._stream())), "barrier")

    for mb in sizes_mb:
        nbytes = mb * 2**20
        n32 = nbytes // 4
        per = (n32 + N - 1) // N
        per = (per + 127) // 128 * 128
        lo, hi = min(rank * per, n32), min(rank * per + per, n32)
        nccl_t = torch.empty(n32, dtype=torch.float32, device=dev).normal_(0, 1e-3)

        def ours_two_shot():
            st = C.c_void_p(K._stream())
            barrier()
            K._check(K.lib.b200_reduce_scatter_f32(buf.ptr_array(), rank, N, C.c_longlong(lo), C.c_longlong(hi - lo),
                                                   C.c_void_p(sumsq.data_ptr()), 0, st), "rs")
            # No barrier here: the push writes slice `rank` of every peer's buffer, and the only reader of that
            # slice (this rank's own reduce-scatter) has already finished on this stream.
            K._check(K.lib.b200_allgather_push_bytes(buf.ptr_array(), rank, N, C.c_longlong(per * 4), 0, st), "ag")
            barrier()

        def ours_one_shot():
            st = C.c_void_p(K._stream())
            barrier()
            K._check(K.lib.b200_allreduce_oneshot_f32(buf.ptr_array(), rank, N, C.c_void_p(out.data_ptr()),
                                                      C.c_longlong(n32), C.c_float(1.0 / N),
                                                      C.c_void_p(sumsq.data_ptr()), 0, st), "oneshot")
            barrier()

        t_nccl = _time(lambda: dist.all_reduce(nccl_t), dev)
        t_two = _time(ours_two_shot, dev) if n32 >= N * 128 else float("nan")
        t_one = _time(ours_one_shot, dev) if mb <= 64 else float("nan")
        bus = 2 * (N - 1) / N * nbytes
        rec = {"bucket_MB": mb, "dtype": "fp32", "n_gpus": N,
               "nccl_ms": round(t_nccl, 4), "nccl_bus_GBps": round(bus / t_nccl / 1e6, 1),
               "two_shot_ms": round(t_two, 4), "two_shot_bus_GBps": round(bus / t_two / 1e6, 1),
               "two_shot_frac_of_link": round(bus / t_two / 1e6 / LINK_GBS, 3),
               "one_shot_ms": round(t_one, 4),
               "one_shot_in_GBps": round((N - 1) * nbytes / t_one / 1e6, 1) if t_one == t_one else None}
        if rank == 0:
            print(json.dumps(rec), flush=True)
    if "--phases" in sys.argv:
        # each phase alone on a 256 MB bucket, by CTA count: inbound (pull) or outbound (push) bytes per GPU per second
        nbytes = 256 * 2**20
        n32 = nbytes // 4
        per = (n32 + N - 1) // N
        lo = rank * per
        moved = (N - 1) * per * 4
        K.lib.b200_allgather_push_bytes.restype = C.c_int
        for ctas in (37, 74, 148, 296, 592):
            def phase(call):
                def run():
                    barrier()
                    K._check(call(C.c_void_p(K._stream())), "phase")
                    barrier()
                return run
            rs_plain = phase(lambda st: K.lib.b200_reduce_scatter_f32(
                buf.ptr_array(), rank, N, C.c_longlong(lo), C.c_longlong(per), None, ctas | 0x10000, st))
            rs_unrolled = phase(lambda st: K.lib.b200_reduce_scatter_f32(
                buf.ptr_array(), rank, N, C.c_longlong(lo), C.c_longlong(per), None, ctas, st))
            ag_pull = phase(lambda st: K.lib.b200_allgather_bytes(buf.ptr_array(), rank, N, C.c_longlong(per * 4), ctas, st))
            ag_push = phase(lambda st: K.lib.b200_allgather_push_bytes(buf.ptr_array(), rank, N, C.c_longlong(per * 4),
                                                                       ctas, st))
            rec = {"phase_sweep_MB": 256, "n_gpus": N, "ctas": ctas}
            for name, fn in (("rs_plain", rs_plain), ("rs_unrolled", rs_unrolled), ("ag_pull", ag_pull),
                             ("ag_push", ag_push)):
                t = _time(fn, dev, reps=6, warmup=2)
                rec[name + "_GBps"] = round(moved / t / 1e6, 1)
            if rank == 0:
                print(json.dumps(rec), flush=True)
    if "--ag" in sys.argv or "--ag-only" in sys.argv:
        # all-gather fused into the consuming GEMM (flagship QKV and gate-up projections, 4096 rows)
        from ..parallel.ag_gemm import GatheredWeight

        for name, Nw, Kw in (("qkv", 15840, 5280), ("mlp.fc", 35840, 5280)):
            gw = GatheredWeight(fabric, Nw, Kw)
            gw.shard.normal_(0, 0.02)
            x = torch.randn(4096, Kw, device=dev).bfloat16()
            torch.cuda.synchronize(dev)
            dist.barrier(device_ids=[dev.index])

            def fused():
                gw.invalidate()
                gw.gemm(x)

            def library():
                gw.gather_only()
                K.gemm_nt(x, gw.full)

            t_fused = _time(fused, dev, reps=6, warmup=2)
            t_lib = _time(library, dev, reps=6, warmup=2)
            gw.gather_only()
            t_gemm = _time(lambda: K.gemm_nt(x, gw.full), dev, reps=6, warmup=2)
            remote = (N - 1) / N * Nw * Kw * 2
            rec = {"ag_gemm": name, "n_gpus": N, "M": 4096, "N": Nw, "K": Kw, "fused_ms": round(t_fused, 3),
                   "gemm_only_ms": round(t_gemm, 3), "nccl_all_gather_then_gemm_ms": round(t_lib, 3),
                   "remote_MB": round(remote / 1e6, 1), "link_floor_ms": round(remote / LINK_GBS / 1e6, 3),
                   "fraction_of_roofline": round(max(t_gemm, remote / LINK_GBS / 1e6) / t_fused, 3)}
            if rank == 0:
                print(json.dumps(rec), flush=True)
            dist.barrier(device_ids=[dev.index])
            gw.close()
    status = K.check_device_status()
    if rank == 0:
        print(json.dumps({"device_status": status}))
    torch.cuda.synchronize(dev)
    ctrl.close()
    buf.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
