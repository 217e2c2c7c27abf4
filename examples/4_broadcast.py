"""Broadcast from ROOT_TEMP (default 0).

Run:  python -m mintccl_b200.launch -np 2 examples/4_broadcast.py        (or torchrun, or mpirun with mpi4py)
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

root = int(os.environ.get("ROOT_TEMP", 0))
dev = "cuda" if cuda else "cpu"
want = torch.randn(count, generator=torch.Generator().manual_seed(root))
buf = torch.randn(count, generator=torch.Generator().manual_seed(rank)).to(dev)
before = buf.clone()
m.broadcast(buf, root)
check("equal", torch.equal(buf.cpu(), want))
if st.enabled():   # MINTCCL_TEST_MODE: the same broadcast through torch.distributed (4_broadcast.py:110-126)
    check("oracle", st.compare(rank, "broadcast", buf, st.oracle(comm).broadcast(before, root), exact=True))

if cuda:
    comm.check()
m.shutdown()
sys.exit(0 if ok else 1)
