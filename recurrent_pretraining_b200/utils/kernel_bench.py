"""Micro-benchmarks of the hot kernels on the flagship shapes, reported against the library GEMM and the measured
machine peaks.  ``python -m recurrent_pretraining_b200.utils.kernel_bench [gemm|swiglu|norm|attn|ce|skinny [shape [batch]]|all]``.

Timing: CUDA events on the launching stream after warm-up, L2 flushed between timed launches by writing a 256 MB
buffer, median of the repeats.
"""
from __future__ import annotations

import json
import os
import statistics
import sys

import torch


def _flush(buf):
    buf.zero_()


def time_fn(fn, reps=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        if flush is not None:
            _flush(flush)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def bench_gemm(M=4096, only=None):
    """``only``: run a single named shape (for profiler captures of one kernel)."""
    from ..ops import cuda as C

    E, I, V = 5280, 17920, 65536
    shapes = [("qkv", 3 * E, E), ("attn.proj", E, E), ("mlp.fc", 2 * I, E), ("mlp.proj", E, I), ("adapter", E, 2 * E),
              ("head(4096 rows)", V, E)]
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    rows = []
    for name, N, K in shapes:
        if only and name != only:
            continue
        x = torch.randn(M, K, device="cuda").bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.02).bfloat16()
        dy = torch.randn(M, N, device="cuda").bfloat16()
        g = torch.zeros(N, K, device="cuda")
        fl = 2.0 * M * N * K
        res = {"shape": name, "M": M, "N": N, "K": K}
        for tag, ours, lib in (
            ("fwd", lambda: C.gemm_nt(x, w), lambda: torch.matmul(x, w.t())),
            ("dgrad", lambda: C.gemm_nn(dy, w), lambda: torch.matmul(dy, w)),
            ("wgrad", lambda: C.gemm_tn(dy, x, out=g, accumulate=True), lambda: torch.matmul(dy.t(), x)),
        ):
            C.set_gemm_2cta(True)
            t_ours = time_fn(ours, flush=flush)
            C.set_gemm_2cta(False)
            t_one = time_fn(ours, flush=flush)
            C.set_gemm_2cta(True)
            t_lib = time_fn(lib, flush=flush)
            res[tag] = {"ours_2cta_ms": round(t_ours, 3), "ours_2cta_tflops": round(fl / t_ours / 1e9, 1),
                        "ours_1cta_tflops": round(fl / t_one / 1e9, 1),
                        "cublas_ms": round(t_lib, 3), "cublas_tflops": round(fl / t_lib / 1e9, 1)}
        rows.append(res)
        print(json.dumps(res), flush=True)
        del x, w, dy, g
    assert C.check_device_status() == 0
    return rows


def bench_norm(M=4096, E=5280):
    from ..ops import cuda as C

    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    if M == 4096:
        bench_norm(M=512, E=E)  # the training shape (4096 rows) first, then 8x that: 346 MB per tensor, larger than L2
    M = M * 8
    x = torch.randn(M, E, device="cuda").bfloat16()
    a = torch.randn(M, E, device="cuda").bfloat16()
    w = torch.ones(E, device="cuda")
    t = time_fn(lambda: C.rmsnorm_fwd(x, w, 1e-6), flush=flush)
    print(json.dumps({"kernel": "rmsnorm_fwd", "rows": M, "ms": round(t, 3), "GBps": round(2 * x.numel() * 2 / t / 1e6, 1)}))
    t = time_fn(lambda: C.add_rmsnorm_fwd(a, x, w, 1e-6), flush=flush)
    print(json.dumps({"kernel": "add_rmsnorm_fwd", "ms": round(t, 3), "GBps": round(4 * x.numel() * 2 / t / 1e6, 1)}))
    y, rstd = C.rmsnorm_fwd(x, w, 1e-6)
    t = time_fn(lambda: C.rmsnorm_bwd(a, x, w, rstd), flush=flush)
    print(json.dumps({"kernel": "rmsnorm_bwd", "rows": M, "ms": round(t, 3), "GBps": round(3 * x.numel() * 2 / t / 1e6, 1)}))


def bench_swiglu(M=4096, E=5280, I=17920):
    """Gate-up GEMM + SwiGLU: one GEMM with the gate in its epilogue against GEMM followed by the elementwise kernel."""
    from ..ops import cuda as C

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    x = torch.randn(M, E, device="cuda").bfloat16()
    w = (torch.randn(2 * I, E, device="cuda") * 0.02).bfloat16()
    t_fused = time_fn(lambda: C.gemm(x, w, out_mode=C.OUT_SWIGLU), flush=flush)
    t_pair = time_fn(lambda: C.swiglu_fwd(C.gemm_nt(x, w)), flush=flush)
    fl = 2.0 * M * 2 * I * E
    print(json.dumps({"kernel": "gate-up GEMM + SwiGLU", "fused_ms": round(t_fused, 3),
                      "fused_tflops": round(fl / t_fused / 1e9, 1), "gemm_then_swiglu_ms": round(t_pair, 3)}))
    # training forms: the forward also stores the bf16 pre-activation; the down projection's input-gradient GEMM applies
    # the gate's derivative in its epilogue
    t_save = time_fn(lambda: C.linear_swiglu_save(x, w), flush=flush)
    print(json.dumps({"kernel": "gate-up GEMM + SwiGLU + pre-activation store (training forward)",
                      "fused_ms": round(t_save, 3), "fused_tflops": round(fl / t_save / 1e9, 1),
                      "gemm_then_swiglu_ms": round(t_pair, 3)}))
    y, h = C.linear_swiglu_save(x, w)
    wp = (torch.randn(E, I, device="cuda") * 0.02).bfloat16()
    dy = torch.randn(M, E, device="cuda").bfloat16()
    t_d = time_fn(lambda: C.dswiglu_dgrad(dy, wp, h), flush=flush)
    t_dpair = time_fn(lambda: C.swiglu_bwd(C.gemm_nn(dy, wp), h), flush=flush)
    fl2 = 2.0 * M * I * E
    print(json.dumps({"kernel": "down-proj dgrad GEMM + dSwiGLU epilogue", "fused_ms": round(t_d, 3),
                      "fused_tflops": round(fl2 / t_d / 1e9, 1), "gemm_then_swiglu_bwd_ms": round(t_dpair, 3)}))
    assert C.check_device_status() == 0


def bench_ce(T=4096, E=5280, V=65536):
    """Head: linear + cross-entropy with the softmax partials from the head GEMM's epilogue (bf16 logits chunk) against
    the older form (fp32 logits chunk + row kernel).  Both include the two gradient GEMMs."""
    from ..ops import cuda as C

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    x = torch.randn(T, E, device="cuda").bfloat16()
    w = (torch.randn(V, E, device="cuda") * 0.02).bfloat16()
    lab = torch.randint(0, V, (T,), device="cuda")
    fl = 3 * 2.0 * T * V * E
    for tag, fused in (("epilogue partials + ce_finish", True), ("fp32 logits chunk + ce_rows", False)):
        t = time_fn(lambda: C.linear_ce(x, w, lab, 1.0, -100, 0.0, need_grad=True, fused=fused), flush=flush)
        print(json.dumps({"kernel": "linear + cross-entropy, forward + both gradients", "form": tag, "ms": round(t, 3),
                          "tflops": round(fl / t / 1e9, 1)}))
    assert C.check_device_status() == 0


def bench_attn(B=1, S=4096, H=55, D=96):
    """Native tcgen05 attention forward / backward against the library path (SDPA) on the flagship shape."""
    from ..ops import attention as A
    from ..ops import cuda as C

    qkv = torch.randn(B, S, 3 * H * D, device="cuda").bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fl = 4.0 * B * H * S * S * D / 2
    scale = D ** -0.5
    t = time_fn(lambda: A.fwd(qkv, H, H, D, scale), flush=flush)
    o, lse = A.fwd(qkv, H, H, D, scale)
    do = torch.randn_like(o)
    tb = time_fn(lambda: A.bwd(do, qkv, o, lse, H, H, D, scale), flush=flush)
    q, k, v = (x.reshape(B, S, H, D).transpose(1, 2) for x in qkv.split(H * D, dim=-1))
    tl = time_fn(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True), flush=flush)
    tlb = time_fn(lambda: C._attention_bwd_library(do, qkv, H, H, D, scale), flush=flush)
    print(json.dumps({"kernel": "attention", "native_bwd": A.NATIVE_BWD, "fwd_ms": round(t, 3),
                      "fwd_tflops": round(fl / t / 1e9, 1), "bwd_ms": round(tb, 3),
                      "bwd_tflops": round(2.5 * fl / tb / 1e9, 1), "library_fwd_ms": round(tl, 3),
                      "library_fwd_plus_bwd_ms": round(tlb, 3)}))


def bench_skinny(only=None, B=1, iters=20):
    """The decode engine's weight-streaming GEMM (out[B, N] = x W^T computed as W x^T) on the flagship projections,
    inside a CUDA graph of ``iters`` launches over four rotating weight copies (so nothing is served from L2)."""
    from ..engine import decode as D
    from ..ops import cuda as K

    shapes = {"qkv": (15840, 5280), "proj": (5280, 5280), "fc": (35840, 5280), "mlpproj": (5280, 17920)}
    work = torch.zeros(B * 15840, device="cuda")
    err = K.err_word(torch.device("cuda", 0))
    for name, (N, Kd) in shapes.items():
        if only and only != name:
            continue
        Ws = [(torch.randn(N, Kd, device="cuda") * 0.02).bfloat16() for _ in range(4)]
        x = torch.randn(B, Kd, device="cuda").bfloat16()
        out = torch.empty(B, N, dtype=torch.bfloat16, device="cuda")
        wk = work if B * N <= work.numel() else None

        def launch(i):
            rc = D._skinny(x.data_ptr(), Ws[i % 4].data_ptr(), out.data_ptr(), K._ptr(wk), B, N, Kd, Kd, Kd, N, 0,
                           K._stream(), err.data_ptr())
            if rc < 0:
                raise RuntimeError(f"b200_gemm_skinny failed with code {rc}")
            return rc

        for i in range(3):
            mode = launch(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        pdl = os.environ.get("B200_DECODE_PDL", "0") == "1"   # programmatic dependent launch between the launches
        old = D._set_pdl(1) if pdl else 0
        with torch.cuda.graph(g):
            for i in range(iters):
                launch(i)
        if pdl:
            D._set_pdl(old)
        t = time_fn(g.replay, reps=5, warmup=1) / iters
        work.zero_()
        print(json.dumps({"kernel": "skinny_gemm", "shape": name, "batch": B, "N": N, "K": Kd,
                          "path": "stream-K fp32 atomics" if mode == 1 else "bf16 store", "pdl": pdl, "us": round(t * 1e3, 1),
                          "weight_TBps": round(N * Kd * 2 / t / 1e9, 2), "device_status": K.check_device_status()}))


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    if what in ("gemm", "all"):
        bench_gemm(only=sys.argv[2] if len(sys.argv) > 2 else None)
    if what in ("swiglu", "all"):
        bench_swiglu()
    if what in ("norm", "all"):
        bench_norm()
    if what in ("attn", "all"):
        bench_attn()
    if what in ("ce", "all"):
        bench_ce()
    if what in ("skinny", "all"):
        bench_skinny(only=sys.argv[2] if len(sys.argv) > 2 else None, B=int(sys.argv[3]) if len(sys.argv) > 3 else 1)
