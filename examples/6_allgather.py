"""All-gather, temporal and spatial CTA layouts.

Run:  python -m mintccl_b200.launch -np 2 examples/6_allgather.py        (or torchrun, or mpirun with mpi4py)
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
parts = [torch.randn(n, generator=torch.Generator().manual_seed(r)) for r in range(world)]
for mode in ("temporal", "spatial"):
    buf = torch.zeros(world, n, device=dev)
    buf[rank] = parts[rank].to(dev)
    m.allgather(buf, mode=mode)
    check(mode, torch.equal(buf.cpu(), torch.stack(parts)))
    if st.enabled():   # MINTCCL_TEST_MODE: dist.all_gather_into_tensor (6_allgather.py:172-179)
        check("oracle", st.compare(rank, f"allgather {mode}", buf, st.oracle(comm).all_gather(parts[rank].to(dev)), exact=True))

if cuda:
    comm.check()
m.shutdown()
sys.exit(0 if ok else 1)
