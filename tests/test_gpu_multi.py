"""Multi-GPU tests (skipped with fewer than two GPUs): child processes under torch.distributed.run, NVLS off."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode: str, nproc: int = 2, port: int = 29641):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", B200_DEBUG_NORM="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "multi_gpu_worker.py"), mode]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    print("\n".join(l for l in r.stdout.splitlines() if "non-finite" in l))
    print(line)          # shown by pytest when the test fails
    return json.loads(line[len("RESULT "):])


needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


def _check_parity(res, sharded_master: bool = False):
    assert res["status"] == 0, res
    assert res["replicas_identical"], res
    for a, b in zip(res["losses"], res["nccl_losses"]):
        assert abs(a - b) < 0.02 * abs(b) + 0.02, res
    for a, b in zip(res["norms"], res["nccl_norms"]):
        assert abs(a - b) < 0.05 * abs(b) + 1e-3, res
    assert res["param_rel_diff"] < 2e-2, res
    assert res["master_rel_diff"] < 2e-2, res


@needs2
@pytest.mark.parametrize("mode", ["train", "train_ellis", "train_accum"])
def test_p2p_sharded_step_matches_nccl_allreduce(mode):
    """Bucketed reduce-scatter fired from the backward pass + sharded update + bf16 push against NCCL all-reduce +
    replicated update, with the recurrence depths changing from step to step; AdamW, the ELLISAdam flags, and a
    two-micro-batch accumulation window."""
    res = _run(mode)
    _check_parity(res)
    kinds = sorted({b.split(".")[0] for b in res["overlap_fired"]})
    assert kinds == ["coda", "core", "last", "prelude"], res


@needs2
@pytest.mark.parametrize("mode", ["zero3", "zero3_ellis"])
def test_parameter_sharded_step_matches_nccl_allreduce(mode):
    """fp32 masters and optimizer state 1/N per rank, bf16 weights pulled in the forward pass (QKV and gate-up inside
    their first GEMM): same losses, norms and parameters as the replicated path, and less memory."""
    res = _run(mode, port=29649)
    _check_parity(res)
    assert res["ag_weights"] > 0, res
    b = res["bytes"]
    assert b["master"] < 0.6 * b["grad"] and b["moments"] < 0.6 * 2 * b["grad"], res


@needs2
def test_barrier_wait_times_out_and_reports():
    res = _run("timeout", port=29643)
    assert res["status"] == 5  # ERR_WAIT_PEER_FLAG
    assert res["after"] == 8.0


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_p2p_sharded_step_four_ranks():
    _check_parity(_run("train", nproc=4, port=29645))
    _check_parity(_run("zero3", nproc=4, port=29651))


@needs2
def test_all_gather_fused_gemm():
    res = _run("ag_gemm", nproc=min(torch.cuda.device_count(), 4), port=29647)
    assert res["status"] == 0
    for name, case in res["cases"].items():
        assert case["rel_err"] < 2e-2, (name, case)
        assert case["weight_equal"] and case["second_call_equal"], (name, case)


@needs2
def test_fused_one_launch_collectives_on_bf16_buckets():
    """All-reduce (one-shot and sliced), reduce-scatter, all-gather and reduce-scatter + clipped AdamW + push, with the
    handshakes inside the kernels, against fp32 torch sums of the same bf16 buckets."""
    res = _run("collectives", nproc=min(torch.cuda.device_count(), 4), port=29653)
    assert res["status"] == 0, res
    for count, case in res["cases"].items():
        for k in ("allreduce_oneshot0", "allreduce_oneshot1", "reduce_scatter"):
            assert case[k] < 1e-6, (count, case)
        assert case["norm_oneshot0"] < 1e-4 and case["norm_oneshot1"] < 1e-4, (count, case)
        assert case["all_gather"] == 0.0, (count, case)
        assert case["adamw_gnorm"] < 1e-4 and case["adamw_master"] < 1e-5 and case["adamw_shadow"] < 2e-2, (count, case)


@needs2
def test_tensor_parallel_blocks_on_the_cuda_kernels():
    """Two-way tensor parallelism (heads and MLP channels split, NCCL all-reduces) on the bf16 CUDA path: loss and
    gradient shards agree with the unsharded model on the same kernels."""
    res = _run("tensor_parallel", nproc=2, port=29655)
    assert res["status"] == 0, res
    assert abs(res["loss_tp"] - res["loss_full"]) < 5e-3 * abs(res["loss_full"]), res
    for k in ("g_qkv", "g_proj", "g_norm", "g_emb"):
        assert res[k] < 3e-2, res
