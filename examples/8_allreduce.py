"""All-reduce (on the reference's roadmap): one-shot LL128 for small, direct / NVLS for symmetric tensors, ring otherwise.

Run:  python -m mintccl_b200.launch -np 2 examples/8_allreduce.py        (or torchrun, or mpirun with mpi4py)
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
parts = [torch.randn(count, generator=torch.Generator().manual_seed(r)).to(torch.float16) for r in range(world)]
ref = sum(p.float() for p in parts)
buf = parts[rank].clone().to(dev)
m.allreduce(buf)                                             # ordinary tensor: shared with the peers on first use
check("ordinary", torch.allclose(buf.cpu().float(), ref, rtol=1e-2, atol=4e-2))
if st.enabled():   # MINTCCL_TEST_MODE: dist.all_reduce on the same inputs
    check("oracle", st.compare(rank, "allreduce", buf, st.oracle(comm).all_reduce(parts[rank].clone().to(dev)),
                               exact=False, roundings=2 * world))
if cuda:
    sym = comm.symm_empty(count, torch.float16)              # symmetric tensor: direct or NVLS
    sym.copy_(parts[rank])
    torch.cuda.synchronize(); comm.control.barrier()
    comm.allreduce(sym)
    check("symmetric", torch.allclose(sym.cpu().float(), ref, rtol=1e-2, atol=4e-2))

if cuda:
    comm.check()
m.shutdown()
sys.exit(0 if ok else 1)
