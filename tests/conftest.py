import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "baseline")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _torch_checkpoint_stays_torchs():
    """The reference package replaces a private function of ``torch.utils.checkpoint`` when its config module is
    imported (a work-around written for an older torch).  Tests that import it as an oracle must not change how
    activation checkpointing behaves in the tests that follow: put torch's own function back after every test."""
    import torch.utils.checkpoint as ck

    original = _TORCH_CHECKPOINT_GENERATOR
    yield
    if ck._checkpoint_without_reentrant_generator is not original:
        ck._checkpoint_without_reentrant_generator = original


import torch.utils.checkpoint as _ck  # noqa: E402

_TORCH_CHECKPOINT_GENERATOR = _ck._checkpoint_without_reentrant_generator
