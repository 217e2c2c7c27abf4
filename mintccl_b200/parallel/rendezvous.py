"""Control plane: how the rank processes find each other and exchange small Python objects.

The reference uses ``mpi4py.MPI.COMM_WORLD`` for this (pickled send/recv/bcast/barrier, e.g.
common.py:26,32 and 3_sendrecv_buffer.py:98-141).  Here the control plane is an interface with three
implementations, picked in this order by :func:`connect`:

* ``MpiControl``        – mpi4py, when it can be imported and the job was started by an MPI launcher;
* ``TorchDistControl``  – a gloo process group of ``torch.distributed`` (started by torchrun, by
  ``python -m mintccl_b200.launch`` or by ``torch.multiprocessing.spawn``);
* ``SingleControl``     – one process, world size 1.

Only small metadata travels here (handles, routes, sizes); tensor data never does.
"""
from __future__ import annotations

import datetime
import os
import pickle
from typing import Any, List


class ControlPlane:
    rank: int = 0
    world_size: int = 1

    def allgather(self, obj: Any) -> List[Any]:
        raise NotImplementedError

    def bcast(self, obj: Any, root: int = 0) -> Any:
        return self.allgather(obj)[root]

    def barrier(self) -> None:
        self.allgather(None)

    def close(self) -> None:
        pass


class SingleControl(ControlPlane):
    def allgather(self, obj):
        return [obj]


class TorchDistControl(ControlPlane):
    """Object collectives over a gloo group (CPU tensors, works with or without GPUs)."""

    def __init__(self, group=None, timeout_s: float = 120.0):
        import torch.distributed as dist
        self._dist = dist
        self._own_pg = False
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29511")
            dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]),
                                    timeout=datetime.timedelta(seconds=timeout_s))
            self._own_pg = True
        if group is None:
            backend = dist.get_backend()
            if "gloo" in str(backend):
                group = dist.group.WORLD
            else:
                group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
        self.group = group
        self.rank = dist.get_rank(group)
        self.world_size = dist.get_world_size(group)

    def allgather(self, obj):
        out = [None] * self.world_size
        self._dist.all_gather_object(out, obj, group=self.group)
        return out

    def bcast(self, obj, root=0):
        box = [obj]
        self._dist.broadcast_object_list(box, src=self._dist.get_global_rank(self.group, root), group=self.group)
        return box[0]

    def barrier(self):
        self._dist.barrier(group=self.group)

    def close(self):
        if self._own_pg and self._dist.is_initialized():
            self._dist.destroy_process_group()


class MpiControl(ControlPlane):
    def __init__(self, comm=None):
        from mpi4py import MPI  # noqa: WPS433 (optional dependency)
        self.comm = comm if comm is not None else MPI.COMM_WORLD
        self.rank = self.comm.Get_rank()
        self.world_size = self.comm.Get_size()

    def allgather(self, obj):
        return self.comm.allgather(obj)

    def bcast(self, obj, root=0):
        return self.comm.bcast(obj, root=root)

    def barrier(self):
        self.comm.Barrier()


def _mpi_launched() -> bool:
    return any(k in os.environ for k in ("OMPI_COMM_WORLD_SIZE", "PMI_SIZE", "PMIX_RANK"))


def connect(group=None) -> ControlPlane:
    """Pick the control plane for this process (see module docstring for the order)."""
    if group is None and _mpi_launched():
        try:
            return MpiControl()
        except ImportError:
            pass
    try:
        import torch.distributed as dist
        if dist.is_available() and (dist.is_initialized() or ("RANK" in os.environ and "WORLD_SIZE" in os.environ)):
            if dist.is_initialized() or int(os.environ["WORLD_SIZE"]) > 1:
                return TorchDistControl(group)
    except ImportError:
        pass
    return SingleControl()


def local_rank_default(rank: int) -> int:
    """Device index for a rank: LOCAL_RANK if the launcher set it, else the rank itself.

    ``torch.cuda.set_device(i)`` indexes the *visible* devices, so CUDA_VISIBLE_DEVICES needs no special
    handling (the reference's set_gpu, common.py:10-17, indexes the visible list with the values of the
    env list, which is only right when the list is a permutation of 0..n-1).
    """
    v = os.environ.get("LOCAL_RANK")
    return int(v) if v is not None else rank


def dumps(obj) -> bytes:
    return pickle.dumps(obj)
