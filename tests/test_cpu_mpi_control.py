"""The mpi4py control plane (``MpiControl``), exercised without an MPI installation: a stand-in ``mpi4py`` package
whose COMM_WORLD runs over a gloo group is put on the path of two child processes that look MPI-launched
(``OMPI_COMM_WORLD_SIZE``).  The reference's only control plane is mpi4py (common.py:26,32)."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

FAKE_MPI = '''
import datetime, os
import torch.distributed as dist


class _Comm:
    def _init(self):
        if not dist.is_initialized():
            dist.init_process_group("gloo", rank=int(os.environ["OMPI_COMM_WORLD_RANK"]),
                                    world_size=int(os.environ["OMPI_COMM_WORLD_SIZE"]),
                                    init_method="file://" + os.environ["FAKE_MPI_RDZV"],
                                    timeout=datetime.timedelta(seconds=60))

    def Get_rank(self):
        self._init()
        return dist.get_rank()

    def Get_size(self):
        self._init()
        return dist.get_world_size()

    def allgather(self, obj):
        out = [None] * dist.get_world_size()
        dist.all_gather_object(out, obj)
        return out

    def bcast(self, obj, root=0):
        box = [obj]
        dist.broadcast_object_list(box, src=root)
        return box[0]

    def Barrier(self):
        dist.barrier()


COMM_WORLD = _Comm()
'''

WORKER = '''
import os, sys, torch
sys.path.insert(0, os.environ["REPO"])
from mintccl_b200.parallel.rendezvous import connect, MpiControl
from mintccl_b200.parallel.cpu_backend import CpuCommunicator
ctl = connect()
assert isinstance(ctl, MpiControl), type(ctl)
r, n = ctl.rank, ctl.world_size
assert n == 2 and ctl.allgather({"rank": r}) == [{"rank": 0}, {"rank": 1}]
assert ctl.bcast("hello" if r == 1 else None, root=1) == "hello"
ctl.barrier()
comm = CpuCommunicator(control=ctl)                 # the public collectives on top of the MPI control plane
x = torch.full((8,), float(r + 1))
comm.allreduce(x)
assert torch.equal(x, torch.full((8,), 3.0))
print("MPI CONTROL OK", r, flush=True)
'''


def test_mpi_control_plane_with_a_stand_in_mpi4py(tmp_path):
    pkg = tmp_path / "fake" / "mpi4py"
    pkg.mkdir(parents=True)
    (pkg / "__init__.py").write_text("")
    (pkg / "MPI.py").write_text(textwrap.dedent(FAKE_MPI))
    worker = tmp_path / "worker.py"
    worker.write_text(textwrap.dedent(WORKER))
    procs = []
    for r in range(2):
        env = dict(os.environ, OMPI_COMM_WORLD_SIZE="2", OMPI_COMM_WORLD_RANK=str(r), FAKE_MPI_RDZV=str(tmp_path / "rdzv"),
                   REPO=ROOT, PYTHONPATH=str(tmp_path / "fake") + os.pathsep + os.environ.get("PYTHONPATH", ""),
                   CUDA_VISIBLE_DEVICES="")
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            env.pop(k, None)
        procs.append(subprocess.Popen([sys.executable, str(worker)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=180) for p in procs]
    for r, (p, (so, se)) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, se[-2000:]
        assert f"MPI CONTROL OK {r}" in so
