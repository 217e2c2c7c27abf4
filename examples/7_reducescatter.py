"""Reduce-scatter: row `rank` of the [world, n] buffer receives the sum over ranks.

Run:  python -m mintccl_b200.launch -np 2 examples/7_reducescatter.py        (or torchrun, or mpirun with mpi4py)
Uses the GPUs when there are any (native kernels), else the CPU reference backend.  MINTCCL_TEST_COUNT sets
the element count (default 1 Mi here; the reference's default of 64 Mi also works).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mintccl_b200 as m  # noqa: E402
from mintccl_b200.utils import selftest as st  # noqa: E402

rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
cuda = torch.cuda.is_available()
if cuda:
    m.set_gpu(int(os.environ.get("LOCAL_RANK", rank)))
comm = m.init()
count = int(os.environ.get("MINTCCL_TEST_COUNT", 1 << 20))
ok = True


def check(what, cond):
    global ok
    ok = ok and bool(cond)
    print(f"# rank {rank}, {what}: {bool(cond)}", flush=True)

dev = "cuda" if cuda else "cpu"
n = count // world
full = [torch.randn(world, n, generator=torch.Generator().manual_seed(r)).to(torch.float16) for r in range(world)]
buf = full[rank].clone().to(dev)
m.reducescatter(buf)
ref = sum(f.float() for f in full)[rank]
check("close", torch.allclose(buf[rank].cpu().float(), ref, rtol=1e-2, atol=4e-2))
if st.enabled():   # MINTCCL_TEST_MODE: dist.reduce_scatter_tensor on the same inputs (7_reducescatter.py:105-117)
    check("oracle", st.compare(rank, "reducescatter", buf[rank], st.oracle(comm).reduce_scatter(full[rank].clone().to(dev)),
                               exact=False, roundings=2 * world))

if cuda:
    comm.check()
m.shutdown()
sys.exit(0 if ok else 1)
