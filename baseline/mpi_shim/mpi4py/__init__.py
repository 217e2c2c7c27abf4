"""Minimal stand-in for mpi4py, backed by a torch.distributed gloo group.

mpi4py and an MPI launcher are not installed in this image, and the reference library uses
``mpi4py.MPI.COMM_WORLD`` as its control plane (pickled send / recv / bcast / barrier).  This package
provides exactly the calls the reference makes so that its files can run UNMODIFIED under
``python -m torch.distributed.run``; none of mintccl_b200 is involved.
"""
from . import MPI  # noqa: F401
