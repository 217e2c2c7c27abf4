"""Sum-reduce to ROOT_TEMP (fp16, fp32 accumulate, checked against an fp32 oracle).

Run:  python -m mintccl_b200.launch -np 2 examples/5_reduce.py        (or torchrun, or mpirun with mpi4py)
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
parts = [torch.randn(count, generator=torch.Generator().manual_seed(r)).to(torch.float16) for r in range(world)]
buf = parts[rank].clone().to(dev)
m.reduce(buf, root)
ref = sum(p.float() for p in parts)
check("close", rank != root or torch.allclose(buf.cpu().float(), ref, rtol=1e-2, atol=4e-2))
if st.enabled():   # MINTCCL_TEST_MODE: dist.reduce(SUM) on the same inputs (5_reduce.py:138-155)
    theirs = st.oracle(comm).reduce(parts[rank].clone().to(dev), root)
    if rank == root:
        check("oracle", st.compare(rank, "reduce", buf, theirs, exact=False, roundings=2 * world))

if cuda:
    comm.check()
m.shutdown()
sys.exit(0 if ok else 1)
