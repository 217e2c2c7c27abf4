"""The example scripts (one per collective, like the reference's numbered self-tests) on the CPU backend,
started with the package's own launcher."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXAMPLES = sorted(f for f in os.listdir(os.path.join(ROOT, "examples")) if f[0].isdigit())


@pytest.mark.parametrize("script", EXAMPLES)
def test_example_on_cpu(script):
    env = dict(os.environ, MINTCCL_TEST_COUNT="4096", CUDA_VISIBLE_DEVICES="")
    world = "3" if script.startswith("2_") else "2"
    r = subprocess.run([sys.executable, "-m", "mintccl_b200.launch", "-np", world, "--timeout", "120",
                        os.path.join(ROOT, "examples", script)], cwd=ROOT, env=env, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "False" not in r.stdout


@pytest.mark.parametrize("script", [f for f in EXAMPLES if f[0] in "1456789" and not f.startswith("10")])
def test_example_self_test_mode_against_torch_distributed(script):
    """MINTCCL_TEST_MODE=1: every script also runs the torch.distributed equivalent (gloo here, NCCL on GPUs) and
    prints the comparison, like the reference's scripts do against NCCL."""
    env = dict(os.environ, MINTCCL_TEST_COUNT="4096", CUDA_VISIBLE_DEVICES="", MINTCCL_TEST_MODE="1",
               MINTCCL_TEST_VERBOSE="1")
    r = subprocess.run([sys.executable, "-m", "mintccl_b200.launch", "-np", "2", "--timeout", "120",
                        os.path.join(ROOT, "examples", script)], cwd=ROOT, env=env, capture_output=True, text=True, timeout=200)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "vs torch.distributed" in r.stdout and "False" not in r.stdout
    assert "torch.dist   head" in r.stdout          # MINTCCL_TEST_VERBOSE
