"""Real multi-GPU runs (one process per GPU, VMM heap exchange, NVLS when the driver offers it)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(n, extra_env=None, timeout=600):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + n), os.path.join(HERE, "multi_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-4000:]
    assert r.stdout.count("MULTI OK") == n, r.stdout[-4000:]


def test_two_gpus():
    _run(2)


def test_all_gpus():
    n = torch.cuda.device_count()
    if n < 4:
        pytest.skip("needs >= 4 GPUs")
    _run(min(n, 8))


def test_two_gpus_ipc_heap():
    """The cudaMalloc + cudaIpc heap, with the ring taken from a discovered and measured link map
    (MINTCCL_TOPO_DISCOVER / MINTCCL_TOPO_MEASURE) and the pair probe of get_p2p_speed run by rank 0."""
    _run(2, {"MINTCCL_HEAP": "ipc", "MINTCCL_TOPO_DISCOVER": "1", "MINTCCL_TOPO_MEASURE": "1", "MINTCCL_TEST_PROBE": "1"})
