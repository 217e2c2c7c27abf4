"""mintccl_b200: a Blackwell-native intra-node collective communication library.

Python-facing API of huangs0/mintccl (send/recv/sync, broadcast, reduce, allgather, reducescatter,
topology search, timers, ``MINTCCL_*`` knobs) plus allreduce, alltoall and fused GEMM+collective ops,
implemented as hand-written sm_100a CUDA kernels over a symmetric heap that every GPU of the node maps.
"""
from .config import Config, NULL, WARP_SIZE, VECTORIZED_BYTES  # noqa: F401
from .topology import (Topology, Route, Plan, find_route, find_ring, get_topology, get_p2p_speed,  # noqa: F401
                       uniform_topology, ring_plan)
from .utils.timer import Timer  # noqa: F401
from .utils.busbw import algbw_gbs, busbw_gbs  # noqa: F401
from .ops.collectives import (init, shutdown, set_gpu, send, recv, sync, broadcast, reduce, allgather,  # noqa: F401
                              reducescatter, allreduce, alltoall, symm_empty, send_ptr, recv_ptr, get_comm)

__version__ = "0.1.0"


def Communicator(*args, **kwargs):
    """Factory for :class:`mintccl_b200.parallel.comm.Communicator` (imported lazily: it needs CUDA)."""
    from .parallel.comm import Communicator as _C
    return _C(*args, **kwargs)


def emulated(nranks: int, device: int = 0, config=None):
    """A world of ``nranks`` ranks on one GPU in this process (single-GPU testing of multi-rank kernels)."""
    from .parallel.comm import Communicator as _C
    return _C.emulated(nranks, device, config)
