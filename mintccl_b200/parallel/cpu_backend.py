"""CPU reference backend: the public collective API on ``torch.distributed`` gloo.

Runs without a GPU (multi-process, world size > 1) and is the oracle for the CUDA kernels: copies are
bit-exact, reductions accumulate in fp32 and round once.  The reference has no CPU path at all and
checks itself against NCCL on a GPU box only (e.g. 6_allgather.py:170-179).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .rendezvous import ControlPlane, connect


class CpuCommunicator:
    """Same method names and in-place conventions as :class:`mintccl_b200.parallel.comm.Communicator`."""

    def __init__(self, control: Optional[ControlPlane] = None, group=None):
        self.control = control or connect(group)
        self.rank, self.world_size = self.control.rank, self.control.world_size
        self.group = getattr(self.control, "group", None)
        self._pending: list = []
        self.ring = list(range(self.world_size))
        self.emulated = False
        self.nvls = False

    # gloo has no reduce for bf16/fp16 on every build: go through fp32, which is also the oracle we want
    def _sum_fp32(self, t: torch.Tensor) -> torch.Tensor:
        acc = t.detach().to(torch.float32).clone()
        if self.world_size > 1:
            dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.group)
        return acc

    def allreduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, **_) -> None:
        (out if out is not None else x).copy_(self._sum_fp32(x).to(x.dtype))

    @staticmethod
    def _raw(t: torch.Tensor) -> torch.Tensor:
        """Byte view: gloo lacks some 16-bit types, and copies do not care about the element type."""
        return t.view(torch.uint8) if t.is_contiguous() else t.contiguous().view(torch.uint8)

    def allgather(self, buff: torch.Tensor, inp: Optional[torch.Tensor] = None, mode: str = "temporal", **_) -> None:
        mine = self._raw((inp if inp is not None else buff[self.rank]).contiguous()).reshape(-1)
        if self.world_size == 1:
            self._raw(buff[0]).reshape(-1).copy_(mine)
            return
        parts = [torch.empty_like(mine) for _ in range(self.world_size)]
        dist.all_gather(parts, mine, group=self.group)
        for r, p in enumerate(parts):
            self._raw(buff[r]).reshape(-1).copy_(p)

    def reducescatter(self, buff: torch.Tensor, out: Optional[torch.Tensor] = None, mode: str = "temporal", **_) -> None:
        acc = self._sum_fp32(buff)
        (out if out is not None else buff[self.rank]).copy_(acc[self.rank].to(buff.dtype).view_as(buff[self.rank]))

    def broadcast(self, buff: torch.Tensor, root: int = 0, **_) -> None:
        if self.world_size > 1:
            dist.broadcast(self._raw(buff), src=root, group=self.group)

    def reduce(self, buff: torch.Tensor, root: int = 0, out: Optional[torch.Tensor] = None, **_) -> None:
        acc = self._sum_fp32(buff)
        if self.rank == root:
            (out if out is not None else buff).copy_(acc.to(buff.dtype))

    def alltoall(self, inp: torch.Tensor, out: torch.Tensor, **_) -> None:
        if self.world_size == 1:
            out.copy_(inp)
            return
        # gloo all_to_all is not available everywhere: n broadcasts of views are slow but always work
        raw_in = inp.contiguous().view(torch.uint8).view(self.world_size, -1)
        raw_out = out.view(torch.uint8).view(self.world_size, -1)
        for src in range(self.world_size):
            rows = raw_in.clone() if src == self.rank else torch.empty_like(raw_in)
            dist.broadcast(rows, src=src, group=self.group)
            raw_out[src].copy_(rows[self.rank])

    # point to point ----------------------------------------------------------------------------------
    def send(self, buff: torch.Tensor, peer: int, rank: Optional[int] = None) -> None:
        self._pending.append(("send", peer, buff))

    def recv(self, buff: torch.Tensor, peer: int, rank: Optional[int] = None) -> None:
        self._pending.append(("recv", peer, buff))

    def sync(self, **_) -> None:
        """Executes posted transfers.  Sends and receives are matched in posting order per pair."""
        reqs = []
        for kind, peer, buff in self._pending:
            raw = self._raw(buff)
            reqs.append(dist.isend(raw, peer, group=self.group) if kind == "send" else dist.irecv(raw, peer, group=self.group))
        for r in reqs:
            r.wait()
        self._pending.clear()
        self.control.barrier()

    def sendrecv_route(self, route: Sequence[int], src, dst, nbytes=None, **_) -> None:
        route = list(route)
        if self.rank == route[0]:
            dist.send(self._raw(src), route[-1], group=self.group)
        elif self.rank == route[-1]:
            dist.recv(self._raw(dst), route[0], group=self.group)

    def symm_empty(self, shape, dtype=torch.float32) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype)

    def symm_zeros(self, shape, dtype=torch.float32) -> torch.Tensor:
        return torch.zeros(shape, dtype=dtype)

    def symm_free(self, t) -> None:
        pass

    def check(self) -> None:
        pass

    def close(self) -> None:
        self.control.barrier()
