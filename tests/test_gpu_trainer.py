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
