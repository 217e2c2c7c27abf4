"""Reference arm of bench.py.

The reference (huangs0/mintccl) has no installer (``pip install`` of its directory fails: neither setup.py
nor pyproject.toml); its README says to copy the files, which is what ``baseline/_ref`` holds.  Its
control plane is mpi4py, which is not installed; ``baseline/mpi_shim`` provides the few calls it makes on
top of a torch.distributed gloo group so that the files can run unmodified under torchrun.

The arm was run once, on 2 x B200, through the reference's own ``allgather(buff)``: its kernel made an
illegal memory access on the first call (record: ``profiles/reference_arm_fault_2xB200.txt``).  Reading the
code shows why: ``send_ptr`` exports the cudaIpc handle of the allocation that CONTAINS the staging tensor
and drops the tensor's offset inside it (common.py:24-26), and the staging tensor itself is released right
after ``.data_ptr()`` is taken (6_allgather.py:153), so the peer writes through a pointer that does not
point at the staging buffer.  The same pattern is in every collective of the reference (4_broadcast.py:93,
5_reduce.py:112), and on 8 GPUs it deadlocks by its own account (README.md:62-63) with unbounded waits.
A GPU memory fault on a shared machine is not repeated, so this arm reports itself unavailable instead of
launching the reference's GPU code again.
"""
from __future__ import annotations

import json
import os


def main(a) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world < 2:
        why = ("the reference's collectives need at least two ranks (its ring search returns no ring for one "
               "device, topology.py:56-93)")
    else:
        why = ("not run again: on 2 x B200 the reference's own allgather kernel made an illegal memory access on its "
               "first call (record: profiles/reference_arm_fault_2xB200.txt; cause by reading: common.py:24-26 exports "
               "the IPC handle of the containing allocation without the offset, 6_allgather.py:153 frees the staging "
               "tensor before use); on 8 GPUs it deadlocks by its own account (README.md:62-63)")
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
