"""Direct send/recv over a peer-mapped buffer (counterpart of the reference's 1_sendrecv_direct.py).

Run:  python -m mintccl_b200.launch -np 2 examples/1_sendrecv_direct.py        (or torchrun, or mpirun with mpi4py)
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

buf = comm.symm_empty(count, torch.float16) if cuda else torch.empty(count, dtype=torch.float16)
payload = torch.randn(count, generator=torch.Generator().manual_seed(0)).to(torch.float16)
if rank == 0:
    buf.copy_(payload)
if cuda:
    torch.cuda.synchronize(); comm.control.barrier()
    comm.sendrecv_direct(0, 1, buf)          # the receiver pulls; ready/done handshake inside the kernel
else:
    (m.send(buf, 1) if rank == 0 else m.recv(buf, 0)) if rank < 2 else None
    m.sync()
check("equal", rank != 1 or torch.equal(buf.cpu(), payload))
if st.enabled() and rank < 2:   # MINTCCL_TEST_MODE: dist.send / dist.recv of the same payload (1_sendrecv_direct.py:93-107)
    theirs = st.oracle(comm).sendrecv(payload.to(buf.device), 0, 1)
    if rank == 1:
        check("oracle", st.compare(rank, "send/recv", buf, theirs, exact=True))

if cuda:
    comm.check()
m.shutdown()
sys.exit(0 if ok else 1)
