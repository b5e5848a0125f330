"""The whole training entry point on one GPU: train, validate, checkpoint, resume."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "train.py")] + args, env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


def test_train_py_trains_validates_saves_and_resumes_on_gpu(tmp_path):
    base = [f"--config={ROOT}/launch_configs/smoke_1xb200.yaml", f"--out_dir={tmp_path}"]
    out = _run(base + ["--max_steps=8"])
    assert "step       8" in out
    files = sorted(os.listdir(tmp_path / "checkpoints-sane-ddp"))
    assert "step-00000006-smoke-b200_0.pth" in files, files
    out2 = _run(base + ["--max_steps=12"])
    assert "Resumed from" in out2 and "step      12" in out2 and "step       3 " not in out2


def test_reference_production_yaml_runs_on_the_fused_path(tmp_path):
    """The field-compatible copy of the reference's main run (ELLISAdam with update clipping, atan2, running init and
    decoupled decay; sampled recurrence; trapezoid schedule) with the model and data swapped for small synthetic ones: the
    optimizer must take the fused flat path, and the loss must be finite and fall."""
    import re

    out = _run([f"--config={ROOT}/launch_configs/frontier_nebel_512_nodes.yaml", f"--out_dir={tmp_path}",
                "--model_name=smoke-raven-96", "--block_size=256", "--world_batch_size=2", "--micro_batch_size=2",
                "--max_tokens=0", "--max_steps=12", "--warmup_steps=2", "--cooldown_steps=2", "--optim_config.lr=1e-3",
                "--logger_name=none", "--log_step_interval=1", "--eval_step_interval=0", "--save_step_interval=0",
                "--save_last_step=false", "--save_n_min_before_job_done=null", "--tokenizer_path=",
                "--model_overwrite={lockstep_n: true, lockstep_k: true}", "--gradient_checkpointing=false",
                "--data_config={train_data: [{type: rngds, prefix: random}], val_data: [{type: rngds, prefix: random}]}"])
    assert "optimizer ELLISAdam runs on the fused flat-buffer kernels" in out, out[-2000:]
    losses = [float(x) for x in re.findall(r"loss ([0-9.]+) \|", out)]
    assert len(losses) >= 10 and all(l == l and l < 20 for l in losses), losses
