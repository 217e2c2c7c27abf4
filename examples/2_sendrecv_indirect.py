"""Multi-hop send/recv: rank 0 -> last rank through every rank in between (LL128 store-and-forward).

Run:  python -m mintccl_b200.launch -np 2 examples/2_sendrecv_indirect.py        (or torchrun, or mpirun with mpi4py)
Uses the GPUs when there are any (native kernels), else the CPU reference backend.  MINTCCL_TEST_COUNT sets
the element count (default 1 Mi here; the reference's default of 64 Mi also works).
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mintccl_b200 as m  # noqa: E402

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

os.environ["MINTCCL_ROUTE"] = "ring"
dev = "cuda" if cuda else "cpu"
payload = torch.randn(count, generator=torch.Generator().manual_seed(0))
buf = payload.to(dev) if rank == 0 else torch.zeros(count, device=dev)
dst = world - 1
if rank == 0:
    m.send(buf, dst)
elif rank == dst:
    m.recv(buf, 0)
m.sync()                                     # everybody calls it, jump hosts included
check("equal", rank != dst or torch.equal(buf.cpu(), payload))

if cuda:
    comm.check()
m.shutdown()
sys.exit(0 if ok else 1)
