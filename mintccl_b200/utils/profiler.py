"""Capture ranges for external profilers (ncu / nsys ``--capture-range=cudaProfilerApi``, NVTX filters).

The reference brackets its direct send/recv kernel with ``cudaProfilerStart`` / ``cudaProfilerStop`` when called
with ``profile=True`` (1_sendrecv_direct.py:73-79).  Here any stretch of code can be bracketed:

    from mintccl_b200.utils.profiler import profile_range
    with profile_range("allreduce 64 MiB"):
        comm.allreduce(x)

The range synchronises the device on entry and exit so that exactly the enclosed launches fall inside it.  Without
CUDA (CPU reference backend) it does nothing.
"""
from __future__ import annotations

import contextlib
from typing import Iterator, Optional

import torch


@contextlib.contextmanager
def profile_range(name: Optional[str] = None, enabled: bool = True, capture: bool = True) -> Iterator[None]:
    """``capture``: also call cudaProfilerStart/Stop (capture range of ncu / nsys); the NVTX range ``name`` is always
    pushed.  ``enabled=False`` makes the whole thing a no-op (so call sites can keep a ``profile=`` flag)."""
    if not enabled or not torch.cuda.is_available():
        yield
        return
    torch.cuda.synchronize()
    if capture:
        torch.cuda.profiler.start()
    if name:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.synchronize()
        if name:
            torch.cuda.nvtx.range_pop()
        if capture:
            torch.cuda.profiler.stop()
