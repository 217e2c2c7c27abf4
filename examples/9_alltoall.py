"""All-to-all (on the reference's roadmap): row p of the input goes to rank p.

Run:  python -m mintccl_b200.launch -np 2 examples/9_alltoall.py        (or torchrun, or mpirun with mpi4py)
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
n = max(1, count // world)
src = (torch.arange(world * n, dtype=torch.float32).view(world, n) + 1000 * rank)
inp = src.to(dev)
out = comm.symm_empty((world, n), torch.float32) if cuda else torch.empty(world, n)
m.alltoall(inp, out)
want = torch.stack([torch.arange(rank * n, (rank + 1) * n, dtype=torch.float32) + 1000 * p for p in range(world)])
check("equal", torch.equal(out.cpu(), want))
if st.enabled():   # MINTCCL_TEST_MODE: dist.all_to_all_single on the same input
    check("oracle", st.compare(rank, "alltoall", out, st.oracle(comm).all_to_all(inp), exact=True))

if cuda:
    comm.check()
m.shutdown()
sys.exit(0 if ok else 1)
