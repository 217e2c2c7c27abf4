"""Module-level collective API with the reference's call signatures.

``send(buff, peer)`` / ``recv(buff, peer)`` / ``sync()`` (2_sendrecv_indirect.py:96-167),
``broadcast(buff, root)`` (4_broadcast.py:79), ``reduce(buff, root)`` (5_reduce.py:99),
``allgather(buff)`` (6_allgather.py:141), ``reducescatter(buff)`` (7_reducescatter.py:81), plus the
``allreduce`` and ``alltoall`` the reference leaves on its roadmap (README.md:23-24).  All operate in
place on a ``torch.Tensor``, run on the current CUDA stream and return nothing.

They act on a process-wide default communicator created on first use (``init()`` creates it
explicitly).  CUDA tensors use the native kernels; CPU tensors, or a machine without a GPU, use the
gloo reference backend.
"""
from __future__ import annotations

from typing import Optional

import torch

_default = None
_default_cpu = None


def init(group=None, config=None, device: Optional[int] = None, backend: Optional[str] = None):
    """Create the default communicator.  ``backend``: "cuda", "cpu" or None (cuda when available)."""
    global _default, _default_cpu
    use_cuda = backend == "cuda" or (backend is None and torch.cuda.is_available())
    if use_cuda:
        from ..parallel.comm import Communicator
        if _default is None:
            _default = Communicator(device=device, config=config, group=group)
        return _default
    from ..parallel.cpu_backend import CpuCommunicator
    if _default_cpu is None:
        _default_cpu = CpuCommunicator(group=group)
    return _default_cpu


def get_comm(t: Optional[torch.Tensor] = None):
    if t is not None and not t.is_cuda:
        return init(backend="cpu")
    return init()


def shutdown() -> None:
    global _default, _default_cpu
    for c in (_default, _default_cpu):
        if c is not None:
            c.close()
    _default = _default_cpu = None


def set_gpu(rank: int) -> None:
    """Bind this process to the GPU of ``rank`` (common.py:10-17).  Indexes the visible devices."""
    if not torch.cuda.is_available():
        return
    if rank >= torch.cuda.device_count():
        raise ValueError(f"rank {rank} >= available GPUs {torch.cuda.device_count()}")
    torch.cuda.set_device(rank)


def send(buff: torch.Tensor, peer: int) -> None:
    get_comm(buff).send(buff, peer)


_profile_next_sync = False


def recv(buff: torch.Tensor, peer: int, profile: bool = False) -> None:
    """Post a receive.  ``profile=True`` brackets the transfer (which runs inside the next :func:`sync`) with a
    profiler capture range, as 1_sendrecv_direct.py:73-79 does around its kernel."""
    global _profile_next_sync
    _profile_next_sync = _profile_next_sync or bool(profile)
    get_comm(buff).recv(buff, peer)


def sync() -> None:
    """Runs every posted send/recv; all ranks must call it (jump hosts included)."""
    global _profile_next_sync
    c = _default if _default is not None else _default_cpu
    c = c or init()
    if _profile_next_sync and torch.cuda.is_available():
        from ..utils.profiler import profile_range
        _profile_next_sync = False
        with profile_range("mintccl_b200.sync"):
            c.sync()
            torch.cuda.synchronize()
    else:
        _profile_next_sync = False
        c.sync()


def broadcast(buff: torch.Tensor, root: int = 0, **kw) -> None:
    get_comm(buff).broadcast(buff, root, **kw)


def reduce(buff: torch.Tensor, root: int = 0, **kw) -> None:
    get_comm(buff).reduce(buff, root, **kw)


def allgather(buff: torch.Tensor, mode: str = "temporal", **kw) -> None:
    get_comm(buff).allgather(buff, mode=mode, **kw)


def reducescatter(buff: torch.Tensor, mode: str = "temporal", **kw) -> None:
    get_comm(buff).reducescatter(buff, mode=mode, **kw)


def allreduce(buff: torch.Tensor, **kw) -> None:
    get_comm(buff).allreduce(buff, **kw)


def alltoall(inp: torch.Tensor, out: torch.Tensor, **kw) -> None:
    get_comm(inp).alltoall(inp, out, **kw)


def symm_empty(shape, dtype=torch.float32):
    """Tensor in the symmetric heap of the default communicator (enables the direct and NVLS algorithms)."""
    return init().symm_empty(shape, dtype)


def send_ptr(ptr_or_tensor, peer: int = -1):
    """Registration half of the reference's ``send_ptr`` (common.py:22-26): returns the serialisable
    ``(ipc_handle, offset)`` pair of the allocation that contains the pointer."""
    import ctypes as C
    from .. import _native as N
    p = ptr_or_tensor.data_ptr() if isinstance(ptr_or_tensor, torch.Tensor) else int(ptr_or_tensor)
    buf = C.create_string_buffer(64)
    off, size = C.c_uint64(0), C.c_uint64(0)
    N.check(N.lib().mt_ipc_export(p, buf, C.byref(off), C.byref(size)), "ipc_export")
    return buf.raw, off.value


def recv_ptr(handle_and_offset) -> int:
    """Mapping half of the reference's ``recv_ptr`` (common.py:29-38): maps a peer's allocation (cached)
    and returns the device address of the peer's pointer in this process."""
    from .. import _native as N
    handle, off = handle_and_offset
    base = N.lib().mt_ipc_open(handle)
    if not base:
        raise RuntimeError(f"cudaIpcOpenMemHandle failed: {N.last_error()}")
    return base + off
