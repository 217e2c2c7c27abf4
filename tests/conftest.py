import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
# The tests pin down which algorithm the built-in policy picks, so the shipped tuning table (measured choices that
# override the policy per size) stays out of them unless a test loads one itself; child processes inherit this.
os.environ.setdefault("MINTCCL_TUNING_FILE", "none")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `pytest -m gpu`)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        ngpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        ngpu = 0
    skip_gpu = pytest.mark.skip(reason="no CUDA device")
    skip_multi = pytest.mark.skip(reason="needs >= 2 CUDA devices")
    for item in items:
        if "gpu" in item.keywords and ngpu == 0:
            item.add_marker(skip_gpu)
        if "multigpu" in item.keywords and ngpu < 2:
            item.add_marker(skip_multi)


def pytest_sessionstart(session):
    """A fresh checkout has no built library (it is not kept in the history): build it once, for sm_100a, before the
    first test needs it.  nvcc cross-compiles, so this works without a GPU; an existing build is left alone."""
    from mintccl_b200 import _native
    if not _native._LIB_PATH.exists():
        from mintccl_b200 import build
        build.build()
